"""Checkpoints in the reference's formats.

1. Core JSON ``checkpoint.json`` (scirust-core/src/checkpoint.rs:28-134): pretty-printed object
   ``{scirust_version, epoch, step, optimizer_state{learning_rate, step, epoch, m, v, beta1_t,
   beta2_t}, weights{name -> flat f32 list}, metadata}``; ``list_checkpoints`` sorted by epoch.
2. SciAgent directory (scirust-sciagent/src/train/checkpoint.rs:28-157 and cuda_model.rs:1534-1856,
   2227-2350): ``meta.json`` (step, loss, lr, config with the 11 model fields) +
   ``model.safetensors`` with keys sorted; optional ``optimizer.safetensors`` (``embedding.{m,v}``,
   ``final_norm.{m,v}``, ``blocks.{i}.{norm1,wq,wk,wv,wo,norm2,wg,wu,wd}.{m,v}``) + ``optimizer.json``
   (version 4) + ``model_semantics.version`` = 2. Directories are published atomically: written as
   ``.step_N.partial`` and renamed to ``step_N``; ``latest_checkpoint`` sorts by the numeric suffix;
   ``prune`` keeps the newest ``keep_last``; ``best/`` holds the model with ``selection.json``.
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path

import numpy as np
import torch

from .safetensors import load_safetensors, save_safetensors

VERSION = "0.1.0"
MODEL_SEMANTICS_VERSION = 2
OPTIMIZER_STATE_VERSION = 4


# ----------------------------------------------------------------------------- core JSON
def save_checkpoint(directory, weights: dict, opt_state: dict, epoch: int, step: int, metadata: dict | None = None):
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    flat = lambda t: [float(v) for v in torch.as_tensor(t, dtype=torch.float32).reshape(-1).tolist()]  # noqa: E731
    ck = {
        "scirust_version": VERSION,
        "epoch": int(epoch),
        "step": int(step),
        "optimizer_state": {
            "learning_rate": float(opt_state.get("learning_rate", 0.0)),
            "step": int(opt_state.get("step", step)),
            "epoch": int(opt_state.get("epoch", epoch)),
            "m": {k: flat(v) for k, v in opt_state.get("m", {}).items()},
            "v": {k: flat(v) for k, v in opt_state.get("v", {}).items()},
            "beta1_t": float(opt_state.get("beta1_t", 1.0)),
            "beta2_t": float(opt_state.get("beta2_t", 1.0)),
        },
        "weights": {k: flat(v) for k, v in weights.items()},
        "metadata": {str(k): str(v) for k, v in (metadata or {}).items()},
    }
    (d / "checkpoint.json").write_text(json.dumps(ck, indent=2))


def load_checkpoint(directory) -> dict:
    p = Path(directory) / "checkpoint.json"
    try:
        ck = json.loads(p.read_text())
    except json.JSONDecodeError as e:
        raise ValueError(f"{p}: not valid JSON ({e})") from None
    for k in ("scirust_version", "epoch", "step", "optimizer_state", "weights", "metadata"):
        if k not in ck:
            raise ValueError(f"{p}: missing field {k!r}")
    return ck


def list_checkpoints(parent) -> list:
    out = []
    parent = Path(parent)
    if not parent.exists():
        return out
    for d in parent.iterdir():
        if d.is_dir() and (d / "checkpoint.json").exists():
            try:
                out.append((int(load_checkpoint(d)["epoch"]), d))
            except (ValueError, KeyError):
                continue
    out.sort(key=lambda e: e[0])
    return out


# ----------------------------------------------------------------------------- SciAgent directory
def _f32_json(x: float) -> float:
    """meta.json stores fp32 values widened to fp64 (``9.999999747378752e-6`` for 1e-5)."""
    return float(np.float32(x))


def _dump_pretty_sorted(obj) -> str:
    # serde_json's pretty printer: 2-space indent, keys in sorted order, exponent without padding
    s = json.dumps(obj, indent=2, sort_keys=True)
    import re
    return re.sub(r"e([+-])0(\d)", r"e\1\2", s).replace("e+", "e")


def save_sciagent_checkpoint(model, path, step: int, loss: float, lr: float, trainer=None, extra_opt: dict | None = None):
    """Write ``path`` atomically (``.{name}.partial`` then rename)."""
    path = Path(path)
    tmp = path.parent / f".{path.name}.partial"
    if tmp.exists():
        shutil.rmtree(tmp)
    tmp.mkdir(parents=True)
    cfg = model.cfg
    meta = {"step": int(step), "loss": _f32_json(loss), "lr": _f32_json(lr),
            "config": {"vocab_size": cfg.vocab_size, "d_model": cfg.d_model, "n_layers": cfg.n_layers,
                       "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads, "d_ff": cfg.d_ff,
                       "max_seq_len": cfg.max_seq_len, "rope_theta": _f32_json(cfg.rope_theta),
                       "tie_embeddings": bool(cfg.tie_embeddings), "use_bias": bool(cfg.use_bias),
                       "eps": _f32_json(cfg.eps)}}
    (tmp / "meta.json").write_text(_dump_pretty_sorted(meta))
    sd = model.reference_state_dict()
    save_safetensors([(k, sd[k]) for k in sorted(sd)], tmp / "model.safetensors")
    if trainer is not None:
        save_optimizer_state(model, trainer, tmp, extra_opt or {})
    (tmp / "model_semantics.version").write_text(f"{MODEL_SEMANTICS_VERSION}\n")
    if path.exists():
        shutil.rmtree(path)
    os.replace(tmp, path)
    return path


def read_meta(path) -> dict:
    p = Path(path) / "meta.json"
    try:
        m = json.loads(p.read_text())
    except (OSError, json.JSONDecodeError) as e:
        raise ValueError(f"cannot read {p}: {e}") from None
    cfg = m.get("config", {})
    from ..models.sciagent import SciAgentConfig
    config = SciAgentConfig(
        vocab_size=int(cfg.get("vocab_size", 32768)), d_model=int(cfg.get("d_model", 1024)),
        n_layers=int(cfg.get("n_layers", 24)), n_heads=int(cfg.get("n_heads", 16)),
        n_kv_heads=int(cfg.get("n_kv_heads", 4)), d_ff=int(cfg.get("d_ff", 2816)),
        max_seq_len=int(cfg.get("max_seq_len", 8192)), rope_theta=float(cfg.get("rope_theta", 1_000_000.0)),
        tie_embeddings=bool(cfg.get("tie_embeddings", True)), use_bias=bool(cfg.get("use_bias", False)),
        eps=float(cfg.get("eps", 1e-5)))
    return {"step": int(m.get("step", 0)), "loss": float(m.get("loss", 0.0)), "lr": float(m.get("lr", 0.0)),
            "config": config}


def load_sciagent_checkpoint(path, device="cpu", model=None, allow_nonexact: bool | None = None):
    """Returns (model, meta). A directory written with RoPE semantics older than version 2 is
    refused unless ``allow_nonexact`` (or env ``SCIAGENT_ALLOW_NONEXACT_RESUME=1``)."""
    from ..models.sciagent import GQADecoder
    path = Path(path)
    meta = read_meta(path)
    sem = path / "model_semantics.version"
    if sem.exists():
        ver = int(sem.read_text().strip() or 0)
        if allow_nonexact is None:
            allow_nonexact = os.environ.get("SCIAGENT_ALLOW_NONEXACT_RESUME") == "1"
        if ver < MODEL_SEMANTICS_VERSION and not allow_nonexact:
            raise ValueError(f"{path}: model semantics version {ver} < {MODEL_SEMANTICS_VERSION}; "
                             "exact resume is not possible")
    if model is None:
        model = GQADecoder(meta["config"], device=device)
    model.load_reference_state_dict(load_safetensors(path / "model.safetensors"))
    return model, meta


_OPT_NAMES = (("norm1", "rms_attn"), ("norm2", "rms_ffn"), ("wo", "wo"), ("wd", "wd"))


def _optimizer_views(model, flat: torch.Tensor) -> dict:
    """Map the reference's optimizer tensor names onto slices of a flat fp32 buffer."""
    cfg = model.cfg
    qd, kd, ff = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.d_ff

    def seg(name, shape):
        o, n = model.segments[name]
        return flat[o:o + n].view(shape)
    out = {"embedding": seg("embed", (cfg.vocab_size, cfg.d_model)), "final_norm": seg("rms_final", (1, cfg.d_model))}
    if "lm_head" in model.segments:          # untied head: its moments and master weights are state too
        out["lm_head"] = seg("lm_head", (cfg.vocab_size, cfg.d_model))
    for i in range(cfg.n_layers):
        wqkv = seg(f"layers.{i}.wqkv", (cfg.d_model, cfg.qkv_dim))
        wgu = seg(f"layers.{i}.wgu", (cfg.d_model, 2 * ff))
        p = f"blocks.{i}"
        out[f"{p}.wq"], out[f"{p}.wk"], out[f"{p}.wv"] = wqkv[:, :qd], wqkv[:, qd:qd + kd], wqkv[:, qd + kd:]
        out[f"{p}.wg"], out[f"{p}.wu"] = wgu[:, :ff], wgu[:, ff:]
        out[f"{p}.wo"] = seg(f"layers.{i}.wo", (qd, cfg.d_model))
        out[f"{p}.wd"] = seg(f"layers.{i}.wd", (ff, cfg.d_model))
        out[f"{p}.norm1"] = seg(f"layers.{i}.rms_attn", (1, cfg.d_model))
        out[f"{p}.norm2"] = seg(f"layers.{i}.rms_ffn", (1, cfg.d_model))
    return out


def save_optimizer_state(model, trainer, directory, extra: dict):
    directory = Path(directory)
    tensors = []
    mv = {"m": _optimizer_views(model, trainer.m), "v": _optimizer_views(model, trainer.v)}
    for name in sorted(mv["m"]):
        for kind in ("m", "v"):
            tensors.append((f"{name}.{kind}", mv[kind][name].detach().float().cpu().contiguous()))
    save_safetensors(tensors, directory / "optimizer.safetensors")
    # fp32 master weights travel in their own file so that a resumed run continues bit for bit
    mw = _optimizer_views(model, trainer.master)
    save_safetensors([(k, mw[k].detach().float().cpu().contiguous()) for k in sorted(mw)],
                     directory / "master.safetensors")
    c = trainer.cfg
    info = {"version": OPTIMIZER_STATE_VERSION, "step": int(trainer.step), "lr": c.lr, "min_lr": c.min_lr,
            "warmup_steps": c.warmup_steps, "total_steps": c.total_steps, "beta1": c.beta1, "beta2": c.beta2,
            "eps": c.eps, "weight_decay": c.weight_decay, "max_grad_norm": c.max_grad_norm}
    info.update(extra)
    (directory / "optimizer.json").write_text(json.dumps(info, indent=2, sort_keys=True))


def load_optimizer_state(model, trainer, directory) -> dict:
    directory = Path(directory)
    info = json.loads((directory / "optimizer.json").read_text())
    if int(info.get("version", 0)) != OPTIMIZER_STATE_VERSION:
        raise ValueError(f"optimizer state version {info.get('version')} != {OPTIMIZER_STATE_VERSION}")
    sd = load_safetensors(directory / "optimizer.safetensors")
    for kind, flat in (("m", trainer.m), ("v", trainer.v)):
        for name, view in _optimizer_views(model, flat).items():
            view.copy_(sd[f"{name}.{kind}"].reshape(view.shape))
    mpath = directory / "master.safetensors"
    if mpath.exists():
        ms = load_safetensors(mpath)
        for name, view in _optimizer_views(model, trainer.master).items():
            view.copy_(ms[name].reshape(view.shape))
    else:
        trainer.master.copy_(model.flat.float())
    model.flat.copy_(trainer.master.to(torch.bfloat16))
    trainer.step = int(info["step"])
    return info


def latest_checkpoint(directory):
    directory = Path(directory)
    if not directory.exists():
        return None

    def num(d):
        n = d.name
        return int(n[5:]) if n.startswith("step_") and n[5:].isdigit() else 0
    dirs = sorted((d for d in directory.iterdir() if d.is_dir() and not d.name.startswith(".")), key=num)
    if not dirs:
        return None
    last = dirs[-1]
    return last if (last / "meta.json").exists() else None


def prune_checkpoints(directory, keep_last: int) -> list:
    directory = Path(directory)
    steps = sorted((d for d in directory.iterdir() if d.is_dir() and d.name.startswith("step_") and d.name[5:].isdigit()),
                   key=lambda d: int(d.name[5:]))
    removed = []
    for d in steps[:-keep_last] if keep_last > 0 else []:
        shutil.rmtree(d)
        removed.append(d)
    return removed


def save_best(model, directory, step: int, metric: float, metric_name: str = "val_loss"):
    best = Path(directory) / "best"
    sel = best / "selection.json"
    if sel.exists():
        prev = json.loads(sel.read_text())
        if prev.get("metric", float("inf")) <= metric:
            return False
    save_sciagent_checkpoint(model, best, step, metric, 0.0)
    sel.write_text(json.dumps({"step": int(step), "metric": float(metric), "metric_name": metric_name}, indent=2))
    return True
