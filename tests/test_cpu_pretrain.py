"""The pretraining loop: pure-function window order, exact resume, evaluation / best / pruning, the environment harness,
and gradient accumulation."""
import json

import numpy as np
import pytest
import torch

from scirust_b200.io import checkpoint as CK
from scirust_b200.models import GQADecoder, SciAgentConfig
from scirust_b200.train import Trainer, TrainerConfig
from scirust_b200.train import pretrain as P

CFG = SciAgentConfig(vocab_size=256, d_model=32, n_layers=1, n_heads=4, n_kv_heads=2, d_ff=64, max_seq_len=32)


def _tokens(n=4000, seed=0):
    base = np.tile(np.arange(17, 57), n // 40 + 1)[:n]
    noise = np.random.default_rng(seed).integers(0, 3, n)
    return (base + noise).astype(np.int64)


def _trainer(seed=0):
    torch.manual_seed(seed)
    return Trainer(GQADecoder(CFG, device="cpu", seed=seed), TrainerConfig(lr=3e-3, weight_decay=0.0))


def test_window_order_is_a_pure_function_of_the_epoch():
    a, b = list(range(10)), list(range(10))
    P.shuffle_windows(a, 7)
    P.shuffle_windows(b, 7)
    assert a == b and sorted(a) == list(range(10)) and a != list(range(10))
    assert P.epoch_order(range(10), 3, True) == P.epoch_order(range(10), 3, True) != P.epoch_order(range(10), 4, True)
    assert P.epoch_order(range(5), 9, False) == [0, 1, 2, 3, 4]
    one = [5]
    P.shuffle_windows(one, 1)
    assert one == [5]
    assert P.corpus_fnv64(np.array([], dtype=np.int64)) == 0xCBF29CE484222325
    assert P.corpus_fnv64([1, 2, 3]) != P.corpus_fnv64([1, 2, 4])


def test_pretrain_learns_logs_evaluates_and_prunes(tmp_path):
    toks = _tokens()
    tr = _trainer()
    logs = []
    cfg = P.PretrainConfig(base_lr=3e-3, min_lr=3e-4, warmup_steps=5, total_steps=60, seq_len=32, batch_size=4, telemetry_interval=7,
                           log_interval=20, save_interval=20, checkpoint_dir=str(tmp_path / "ck"), val_frac=0.1, eval_interval=30,
                           eval_windows=8, keep_last=2, weight_decay=0.0)
    losses = P.pretrain(tr, toks, cfg, log=logs.append)
    assert len(losses) == 60 and losses[-1] < 0.6 * losses[0] and tr.step == 60
    assert sum("tok/s" in l for l in logs) == 3 and sum("validation loss" in l for l in logs) == 2 and any("held-out validation" in l for l in logs)
    kept = sorted(p.name for p in (tmp_path / "ck").iterdir())
    assert kept == ["best", "step_40", "step_60"]                                   # keep_last = 2, best/ lives apart
    sel = json.loads((tmp_path / "ck" / "best" / "selection.json").read_text())
    assert sel["step"] in (30, 60) and sel["metric"] > 0
    assert P.pretrain(tr, toks[:20], cfg, log=logs.append) == [] and "shorter than a single window" in logs[-1]
    with pytest.raises(P.PretrainError, match="load the optimizer state first"):
        P.pretrain(_trainer(), toks, P.PretrainConfig(total_steps=10, start_step=5, seq_len=32, checkpoint_dir=str(tmp_path / "x")))


def _interrupt_after(trainer, toks, cfg, stop_step):
    """Run the loop and kill it right after the checkpoint of ``stop_step`` is on disk (as a pre-empted job would be)."""
    class _Stop(Exception):
        pass
    orig = CK.save_sciagent_checkpoint

    def saving(model, path, step, loss, lr, trainer=None, extra_opt=None):
        out = orig(model, path, step, loss, lr, trainer=trainer, extra_opt=extra_opt)
        if step == stop_step:
            raise _Stop()
        return out
    CK.save_sciagent_checkpoint = saving
    try:
        P.pretrain(trainer, toks, cfg, log=lambda *_: None)
    except _Stop:
        return
    finally:
        CK.save_sciagent_checkpoint = orig
    raise AssertionError("the run was not interrupted")


def test_resume_is_bit_identical_to_the_uninterrupted_run(tmp_path):
    toks = _tokens(3000, 1)
    common = dict(base_lr=2e-3, min_lr=2e-4, warmup_steps=3, total_steps=24, seq_len=32, batch_size=3, telemetry_interval=5,
                  log_interval=0, weight_decay=0.0, shuffle=True)
    whole = _trainer(4)
    all_losses = P.pretrain(whole, toks, P.PretrainConfig(checkpoint_dir=str(tmp_path / "a"), **common), log=lambda *_: None)
    _interrupt_after(_trainer(4), toks, P.PretrainConfig(checkpoint_dir=str(tmp_path / "b"), save_interval=10, **common), 10)
    last = CK.latest_checkpoint(tmp_path / "b")
    assert last is not None and last.name == "step_10"
    model2, meta = CK.load_sciagent_checkpoint(last, device="cpu")
    second = Trainer(model2, TrainerConfig(lr=2e-3, weight_decay=0.0))
    CK.load_optimizer_state(model2, second, last)
    cfg2 = P.PretrainConfig(checkpoint_dir=str(tmp_path / "b"), start_step=int(meta["step"]), **common)
    resumed = P.pretrain(second, toks, cfg2, log=lambda *_: None)
    assert resumed == all_losses[10:]                                               # the same next windows, the same bits
    assert torch.equal(second.model.flat, whole.model.flat) and torch.equal(second.m, whole.m) and second.step == 24


def test_environment_harness(tmp_path):
    text = tmp_path / "corpus"
    text.mkdir()
    (text / "a.txt").write_bytes(b"the quick brown fox jumps over the lazy dog\n" * 60)
    logs = []
    env = {"SCIAGENT_TEXT": str(text), "SCIAGENT_CKPT": str(tmp_path / "ck"), "SCIAGENT_STEPS": "6", "SCIAGENT_SEQ": "32",
           "SCIAGENT_BATCH": "2", "SCIAGENT_SAVE": "3", "SCIAGENT_TELEMETRY": "2", "SCIAGENT_KEEP": "5", "SCIAGENT_CONFIG": "debug"}
    cfg = P.PretrainConfig.from_env(env)
    assert (cfg.total_steps, cfg.seq_len, cfg.batch_size, cfg.save_interval, cfg.save_interval_seconds, cfg.keep_last) == (6, 32, 2, 3, 0, 5)
    assert P.PretrainConfig.from_env({}).save_interval_seconds == 6 * 3600 and P.PretrainConfig.from_env({"SCIAGENT_SHUFFLE": "0"}).shuffle is False
    assert P.run_from_env({**env, "SCIAGENT_PREFLIGHT_ONLY": "1"}, log=logs.append, device="cpu") == 0
    assert logs[-1].startswith("SCIAGENT_PREFLIGHT_OK") and not (tmp_path / "ck").exists()
    n_tok = 60 * 44 + 1
    assert f"corpus_tokens={n_tok}" in logs[-1]
    assert P.run_from_env({**env, "SCIAGENT_EXPECT_CORPUS_TOKENS": "5"}, log=logs.append, device="cpu") == 3
    assert P.run_from_env({**env, "SCIAGENT_REQUIRE_FRESH": "1", "SCIAGENT_MAX_TOKENS": "100"}, log=logs.append, device="cpu") == 3
    assert P.run_from_env(env, log=logs.append, device="cpu") == 0
    assert sorted(p.name for p in (tmp_path / "ck").iterdir()) == ["step_3", "step_6"] and any(l.startswith("done: 6 steps") for l in logs)
    assert P.run_from_env({**env, "SCIAGENT_REQUIRE_FRESH": "1"}, log=logs.append, device="cpu") == 3       # directory is no longer empty
    logs.clear()
    assert P.run_from_env({**env, "SCIAGENT_STEPS": "8"}, log=logs.append, device="cpu") == 0                 # resumes from step 6
    assert any("resumed from" in l and "step 6" in l for l in logs) and any(l.startswith("done: 2 steps") for l in logs)
    shards = tmp_path / "shards"
    shards.mkdir()
    np.array([1, 2, 999999, 4] * 50, dtype="<u4").tofile(shards / "s.bin")
    assert P.run_from_env({"SCIAGENT_SHARDS": str(shards), "SCIAGENT_CKPT": str(tmp_path / "ck2"), "SCIAGENT_CONFIG": "debug",
                           "SCIAGENT_SEQ": "16"}, log=logs.append, device="cpu") == 3
    assert "another vocabulary" in logs[-1]
    from scirust_b200 import cli
    assert cli.run(["pretrain", "--text", str(text), "--ckpt", str(tmp_path / "ck3"), "--config", "debug", "--seq", "32", "--preflight-only",
                    "--device", "cpu"]) == 0
    assert SciAgentConfig.preset("byte").vocab_size == 256 and SciAgentConfig.preset("code350m").n_layers == 24 and SciAgentConfig.preset("demo").vocab_size == 512


def test_gradient_accumulation_equals_the_big_batch_step():
    torch.manual_seed(0)
    batch = torch.randint(0, 256, (8, 33))
    a, b = _trainer(2), _trainer(2)
    la = a.train_step(batch)
    lb = b.train_step_accumulated([batch[:2], batch[2:4], batch[4:6], batch[6:]])
    assert float(la) == pytest.approx(float(lb), rel=1e-3)
    rel = float((a.model.flat.float() - b.model.flat.float()).norm() / a.model.flat.float().norm())
    assert rel < 2e-3 and a.step == b.step == 1
    assert a.grad_norm() == pytest.approx(b.grad_norm(), rel=2e-2)
    with pytest.raises(ValueError):
        b.train_step_accumulated([])


def test_bench_record_schema_and_capability_registry(tmp_path):
    from scirust_b200.utils import bench_schema as BS
    from scirust_b200.utils import capability_registry as CR
    r = BS.BenchRecord("gemm", "B8xS2048", "tcgen05", 7, "tflops", 1434.0)
    assert json.loads(r.to_json_row()) == {"kernel": "gemm", "dataset": "B8xS2048", "method": "tcgen05", "seed": 7, "metric": "tflops", "value": 1434.0}
    full = (r.with_ci(BS.ConfidenceInterval(1400.0, 1460.0, 0.95)).with_cert(BS.Certificate("fixed k order", determinism="bitwise"))
            .with_prereg(BS.Preregistration("a" * 64, "b" * 64, True, "ratio >= 0.85"))
            .with_evidence(BS.ScientificEvidence("empirical_validation", "supports", "measured on one B200")))
    assert full.is_confirmatory() and not r.is_confirmatory() and "bound_ulps" not in full.to_json_row()
    assert not r.with_prereg(BS.Preregistration("a", "b", False)).is_confirmatory()
    back = BS.parse_jsonl(BS.to_jsonl([r, full]) + "\n")
    assert back == [r, full]
    BS.write_jsonl(tmp_path / "rows.jsonl", [full])
    assert BS.parse_jsonl((tmp_path / "rows.jsonl").read_text()) == [full]
    assert BS.ScientificEvidence("rejection_criterion", "rejects", "x").is_negative_result()
    for bad in ('{"kernel":"k"}', '{"kernel":"k","dataset":"d","method":"m","seed":-1,"metric":"x","value":1}',
                '{"kernel":"k","dataset":"d","method":"m","seed":1,"metric":"x","value":"fast"}', "[1,2]", "{not json",
                '{"kernel":"k","dataset":"d","method":"m","seed":1,"metric":"x","value":1,"extra":2}',
                '{"kernel":"k","dataset":"d","method":"m","seed":1,"metric":"x","value":1,"evidence":{"kind":"empirical_validation","disposition":"supports","statement":" "}}'):
        with pytest.raises(BS.BenchSchemaError):
            BS.parse_jsonl(bad)
    line = json.dumps({"metric": "train_tokens_per_s", "value": 599600.0, "unit": "tok/s", "ms_per_step": 27.32, "dtype": "bf16", "data": "synthetic",
                       "config": {"model": "gqa_12l", "global_batch": 8, "seq_len": 2048, "parallelism": "dp1"},
                       "e2e": {"value": 580700.0, "unit": "tok/s"}})
    rows = BS.from_bench_line(line, seed=1234)
    assert [x.value for x in rows] == [599600.0, 580700.0, 27.32] and rows[1].method.endswith(":e2e") and rows[0].kernel == "gqa_12l"
    CR.clear()
    assert CR.capability_summary() == "none"
    caps = CR.register_default_capabilities()
    doms = [c.domain for c in caps]
    assert doms == sorted(doms, key=CR.DOMAINS.index) and {"cpu-simd", "cpu-native", "cuda"} <= set(doms)
    assert next(c for c in caps if c.domain == "cpu-native").available is True
    cu = next(c for c in caps if c.name == "kernels")
    assert cu.available is (True if torch.cuda.is_available() else False)
    CR.register_capability(CR.Capability("cuda", "kernels", "replaced", None))
    assert sum(c.name == "kernels" for c in CR.capabilities("cuda")) == 1 and "cuda:kernels?" in CR.capability_summary()
    with pytest.raises(ValueError):
        CR.register_capability(CR.Capability("tpu", "x"))
    assert next(c for c in CR.register_default_capabilities(probe=False) if c.domain == "cpu-native").available is None
