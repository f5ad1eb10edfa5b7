"""Supervised fine-tuning (prompt format, padding and prompt masking, learning), held-out evaluation, byte shards."""
import json
import math

import numpy as np
import pytest
import torch

from scirust_b200.data.corpus import ShardLoader, byte_shard, load_byte_shard
from scirust_b200.models import GQADecoder, SciAgentConfig
from scirust_b200.tokenizer import BpeTrainer
from scirust_b200.train import evaluate as EV
from scirust_b200.train import sft as SFT


def _tokenizer():
    return BpeTrainer(80, min_frequency=1).train(["user: say hello world assistant: hello world", "user: say moon assistant: moon"])


def test_sft_prompt_format_batching_and_masking(tmp_path):
    tok = _tokenizer()
    ex = SFT.SftExample("say hello", "hello")
    tokens, start = SFT.format_sft_prompt(ex, tok, True)
    bos, eos = tok.special_id("<bos>"), tok.special_id("<eos>")
    assert tokens[0] == bos == 1 and tokens[-1] == eos == 2 and tokens.count(bos) == 2 and tokens.count(eos) == 2
    assert tok.decode(tokens[start:-1]) == "hello" and SFT.format_sft_prompt(ex, tok) == tokens
    inp, tgt = SFT.sft_batch([ex, SFT.SftExample("say moon", "moon moon")], tok, 48)
    assert inp.shape == tgt.shape == (2, 48)
    n = len(tokens) - 1
    assert inp[0, :n].tolist() == tokens[:-1] and int(inp[0, n:].abs().sum()) == 0
    live = torch.nonzero(tgt[0] >= 0).reshape(-1).tolist()
    assert live == list(range(start - 1, n)) and tgt[0, live].tolist() == tokens[start:]      # only the response teaches
    full = SFT.sft_batch([ex], tok, 48, mask_prompt=False)[1]
    assert int((full >= 0).sum()) == n
    short = SFT.sft_batch([ex], tok, 6)                                                        # truncation keeps the shapes
    assert short[0].shape == (1, 6) and short[0][0].tolist() == tokens[:6]
    p = tmp_path / "sft.jsonl"
    p.write_text(json.dumps({"instruction": "say hello", "output": "hello",
                             "tool_calls": [{"name": "calc", "params": {"x": "1"}}, {"bad": 1}]}) + "\n\n"
                 + json.dumps({"instruction": 5, "output": "moon"}) + "\n")
    ds = SFT.SftDataset.from_jsonl(p)
    assert len(ds) == 2 and ds.examples[0].tool_calls[0].name == "calc" and ds.examples[0].tool_calls[0].params == [("x", "1")]
    assert len(ds.examples[0].tool_calls) == 1 and ds.examples[1].instruction == "" and not ds.is_empty()
    p.write_text("{not json}\n")
    with pytest.raises(ValueError):
        SFT.SftDataset.from_jsonl(p)


def test_sft_training_learns_the_responses():
    tok = _tokenizer()
    torch.manual_seed(0)
    cfg = SciAgentConfig(vocab_size=(tok.vocab_size() + 7) // 8 * 8, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=64,
                         max_seq_len=64)
    model = GQADecoder(cfg, device="cpu")
    ds = SFT.SftDataset([SFT.SftExample("say hello world", "hello world"), SFT.SftExample("say moon", "moon")])
    logs = []
    hist = SFT.sft_train(model, ds, tok, 1e-2, 200, 2, 48, log=logs.append)
    assert hist[-1] < 0.3 * hist[0] and hist[-1] < 0.5 and any("avg loss" in l for l in logs)
    # greedy continuation of the prompt reproduces the response
    tokens, start = SFT.format_sft_prompt(ds.examples[1], tok, True)
    seq = tokens[:start]
    with torch.no_grad():
        for _ in range(len(tokens) - start):
            seq.append(int(model(torch.tensor([seq]))[0].argmax()))       # forward without targets: logits of the last position
    assert tok.decode(seq[start:-1]) == "moon" and seq[-1] == tok.special_id("<eos>")


def test_heldout_evaluation_and_byte_shards(tmp_path):
    src = tmp_path / "src"
    (src / "sub").mkdir(parents=True)
    (src / "a.rs").write_bytes(b"fn main() {}\n" * 20)
    (src / "sub" / "b.rs").write_bytes(b"struct S;\n" * 30)
    (src / "c.txt").write_bytes(b"ignored")
    n, paths = byte_shard([src], tmp_path / "raw", "rs", recursive=True, tokens_per_shard=300)
    total = 13 * 20 + 10 * 30 + 2
    assert n == 2 and [p.name for p in paths] == ["shard_0000.bin", "shard_0001.bin"]
    toks = np.concatenate([load_byte_shard(p) for p in paths])
    assert toks.size == total and int((toks == 0xFF).sum()) == 2 and bytes(toks[:12].astype(np.uint8)) == b"fn main() {}"
    assert byte_shard([src], tmp_path / "none", "rs", recursive=False)[0] == 0            # directories need --recursive
    assert byte_shard([src / "a.rs", src / "sub" / "b.rs"], tmp_path / "one", max_files=1)[0] == 1
    n32, p32 = byte_shard([src], tmp_path / "u32", "rs", recursive=True, tokens_per_shard=10_000, as_u32=True)
    loader = ShardLoader()
    loader.load_dir(tmp_path / "u32")
    assert loader.total_tokens() == total and np.array_equal(loader.tokens(), toks)
    torch.manual_seed(0)
    cfg = SciAgentConfig(vocab_size=256, d_model=32, n_layers=1, n_heads=4, n_kv_heads=2, d_ff=64, max_seq_len=32)
    model = GQADecoder(cfg, device="cpu")
    rep = EV.evaluate_shards(model, tmp_path / "u32", batch_size=4)
    assert rep.tokens == total and rep.sequences == (total - 1) // 32 and rep.batches == rep.sequences // 4
    assert rep.mean_loss == pytest.approx(math.log(256), abs=0.5) and rep.perplexity == pytest.approx(math.exp(rep.mean_loss))
    again = EV.evaluate_shards(model, tmp_path / "u32", batch_size=4)
    assert again == rep                                                                   # deterministic measurement
    capped = EV.evaluate_shards(model, tmp_path / "u32", batch_size=4, max_batches=2)
    assert capped.batches == 2
    # training on the shards lowers the held-out number
    from scirust_b200.train import Trainer, TrainerConfig
    tr = Trainer(model, TrainerConfig(lr=3e-3, weight_decay=0.0))
    data = torch.from_numpy(loader.tokens().astype(np.int64))
    for s in range(40):
        i = (s * 33) % (total - 4 * 33)
        tr.train_step(data[i:i + 4 * 33].reshape(4, 33))
    assert EV.evaluate_shards(model, tmp_path / "u32", batch_size=4).mean_loss < rep.mean_loss - 1.0


def test_cli_data_finetune_eval_and_assurance_commands(tmp_path, capsys):
    from scirust_b200 import cli
    from scirust_b200.io import checkpoint as CK
    src = tmp_path / "src"
    src.mkdir()
    (src / "a.rs").write_bytes(b"fn main() { println!(\"hi\"); }\n" * 40)
    assert cli.run(["byte-shard", "-i", str(src), "-o", str(tmp_path / "sh"), "--recursive", "--u32", "--tokens-per-shard", "500"]) == 0
    out = capsys.readouterr().out
    assert "Total files: 1" in out and "shard_0002.bin" in out
    torch.manual_seed(0)
    cfg = SciAgentConfig(vocab_size=256, d_model=32, n_layers=1, n_heads=4, n_kv_heads=2, d_ff=64, max_seq_len=32)
    CK.save_sciagent_checkpoint(GQADecoder(cfg, device="cpu"), tmp_path / "ck" / "step_1", 1, 5.5, 1e-3)
    assert cli.run(["eval-shards", "--checkpoint", str(tmp_path / "ck" / "step_1"), "--data-dir", str(tmp_path / "sh"),
                    "--batch-size", "4", "--device", "cpu"]) == 0
    out = capsys.readouterr().out
    assert "perplexity" in out and "step 1" in out
    tok = _tokenizer()
    tok.save_json(tmp_path / "bpe.json")
    (tmp_path / "sft.jsonl").write_text(json.dumps({"instruction": "say moon", "output": "moon"}) + "\n")
    assert cli.run(["sft", "--data", str(tmp_path / "sft.jsonl"), "--tokenizer", str(tmp_path / "bpe.json"), "--epochs", "3",
                    "--batch-size", "1", "--max-seq-len", "40", "--device", "cpu", "--out", str(tmp_path / "sft_out")]) == 0
    assert "avg loss" in capsys.readouterr().out and (tmp_path / "sft_out" / "model.safetensors").exists()
    (tmp_path / "empty.jsonl").write_text("\n")
    assert cli.run(["sft", "--data", str(tmp_path / "empty.jsonl"), "--tokenizer", str(tmp_path / "bpe.json"), "--device", "cpu"]) == 3
    assert cli.run(["sft", "--data", str(tmp_path / "missing.jsonl"), "--tokenizer", str(tmp_path / "bpe.json")]) == 2
    capsys.readouterr()
    expect = {"robust": "branch and bound", "watermark": "wrong key", "prune": "wanda", "conformal-sets": "RAPS", "fuse": "fused kernels"}
    for cmd, needle in expect.items():
        assert cli.run([cmd]) == 0
        assert needle in capsys.readouterr().out
    assert cli.run(["dp-sgd", "--steps", "5"]) == 0 and "epsilon" in capsys.readouterr().out
    assert cli.run(["ensemble", "--steps", "50", "--members", "3"]) == 0 and "outside the data" in capsys.readouterr().out
    assert cli.run(["robust", "--eps", "-1"]) == 2 and cli.run(["prune", "--sparsity", "2"]) == 2
    assert cli.run(["dp-sgd", "--noise", "0"]) == 3
