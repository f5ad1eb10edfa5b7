"""Child of the tensor-parallel inference tests: every rank builds the same small decoder, serves it
through ``TPInferenceEngine`` and compares prefill logits and greedy tokens with the single-rank
engine (rank-local, full weights). Runs on CPU under gloo or on GPUs under NCCL."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from scirust_b200.models import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.models.infer import InferenceEngine, teacher_forced_logits  # noqa: E402
from scirust_b200.models.infer_tp import TPInferenceEngine  # noqa: E402


def main():
    use_cuda = os.environ.get("SB_TEST_DEVICE", "cpu") == "cuda"
    backend = os.environ.get("SB_TP_BACKEND", "fused")
    quant = os.environ.get("SB_TP_QUANT") or None
    rank = int(os.environ["RANK"])
    if use_cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    W = dist.get_world_size()
    cfg = SciAgentConfig(vocab_size=512, d_model=512, n_layers=2, n_heads=8, n_kv_heads=int(os.environ.get("SB_TP_KV", "4")),
                         d_ff=512, max_seq_len=256)
    model = GQADecoder(cfg, device=dev, seed=3, init_std=0.08)
    B, P, NEW = (2, 24, 6) if not use_cuda else (int(os.environ.get("SB_TP_BATCH", "2")), 40, 8)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    single = InferenceEngine(model, quant=quant, max_batch=B, max_seq=P + NEW + 1, page=16)
    ref_logits = single.prefill(prompts).float().cpu().clone()
    ref_tokens = single.generate(prompts, NEW).cpu()
    tp = TPInferenceEngine(model, quant=quant, max_batch=B, max_seq=P + NEW + 1, page=16, backend=backend)
    logits = tp.prefill(prompts).float().cpu().clone()
    err = (logits - ref_logits).abs().max().item()
    scale = ref_logits.abs().max().item()
    # int8: a rank quantises its own weight shard and (W8A8) its own share of the activations, so the two engines
    # differ by quantisation noise, not by rounding order
    assert err <= (1e-1 if quant else 3e-2) * max(1.0, scale), f"rank {rank}: prefill logits differ by {err} (scale {scale})"
    tokens = tp.generate(prompts, NEW).cpu()
    again = tp.generate(prompts, NEW).cpu()
    assert torch.equal(tokens, again), "tensor-parallel decode is not repeatable"
    # all ranks must emit identical tokens (the reductions add in rank order on every rank)
    tok_dev = tokens.to(dev)                      # collectives take tensors of the group's device only
    gathered = [torch.empty_like(tok_dev) for _ in range(W)]
    dist.all_gather(gathered, tok_dev)
    for t in gathered:
        assert torch.equal(t.cpu(), tokens), "ranks disagree on the generated tokens"
    # teacher forcing: both engines are fed the single-rank engine's tokens, so every decode step (GEMV, the fused
    # GEMV + all-reduce, paged attention, vocabulary-parallel head) is compared on identical inputs, logits against
    # logits, instead of counting how long two greedy runs stay on the same prefix
    ref_steps = teacher_forced_logits(single, prompts, ref_tokens).cpu()
    tp_steps = teacher_forced_logits(tp, prompts, ref_tokens).cpu()
    step_err = (tp_steps - ref_steps).abs().amax(dim=(0, 2))
    step_scale = ref_steps.abs().amax(dim=(0, 2)).clamp(min=1.0)
    # int8: a rank quantises its own shard, so the row-parallel matrices get other per-column scales than the
    # unsharded matrix and the two engines differ by quantisation noise, not by rounding order
    tol = 1e-1 if quant else 3e-2
    assert bool((step_err <= tol * step_scale).all()), f"rank {rank}: per-step logits differ: {step_err.tolist()}"
    if use_cuda and backend == "fused" and tp.gemv_chan is not None:
        # the GEMV that performs its own all-reduce must give the bits of the GEMV + stand-alone all-reduce pair
        os.environ["SB_TP_FUSED_GEMV"] = "0"
        tp2 = TPInferenceEngine(model, quant=quant, max_batch=B, max_seq=P + NEW + 1, page=16, backend=backend)
        os.environ.pop("SB_TP_FUSED_GEMV")
        assert tp2.gemv_chan is None
        pair_steps = teacher_forced_logits(tp2, prompts, ref_tokens).cpu()
        assert torch.equal(pair_steps, tp_steps), "fused GEMV + all-reduce differs from the two-kernel path"
        tp2.close()
    if use_cuda and getattr(tp, "amax_chan", None) is not None and B <= 8:
        # the vocabulary-parallel head that exchanges (value, column) candidates inside the GEMV launch must emit the
        # tokens of the path that gathers the logit shards and runs the stand-alone arg-max
        assert tp._fused_argmax_ok(B)
        tp.fused_argmax = False
        unfused = tp.generate(prompts, NEW).cpu()
        tp.fused_argmax = True
        assert torch.equal(unfused, tokens), "fused LM head + arg-max differs from gather + arg-max"
    match = (tokens == ref_tokens).float().mean().item()       # reported, not asserted
    if use_cuda:
        from scirust_b200.ops import _lib
        _lib.check_status(dev)
        torch.cuda.synchronize()
    tp.close()
    dist.barrier()
    if rank == 0:
        print(f"TP_INFER_OK world={W} backend={tp.backend} logits_err={err:.4f} token_match={match:.2f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
