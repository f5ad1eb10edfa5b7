#!/usr/bin/env python
"""Inference benchmark at Llama-3-8B shape (32 layers, d 4096, 32 query / 8 KV heads, head_dim 128,
SwiGLU 14336, vocab 128256, RoPE theta 5e5, random-init bf16 weights): prefill of ``--prompt``
synthetic tokens, then greedy decode of ``--new`` tokens with a paged bf16 KV cache, at batch
``--batch``; bf16 or int8 per-output-channel weights. Reports p50 time-to-first-token (prefill +
first arg-max + device->host copy of the token) and decode tokens/s (CUDA-graph replay, device-side
token feedback), timed with CUDA events.

    python examples/infer_bench.py --batch 1 --quant none
    python examples/infer_bench.py --model gqa_12l --batch 16 --prompt 512 --new 64
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/infer_bench.py --tp 4

With ``--tp N`` (launched as N ranks) the model is served tensor-parallel over N GPUs; times are the
maximum over ranks. ``--comm nccl`` swaps the peer-memory collectives for NCCL (the baseline).
"""
import argparse
import json
import statistics
import sys
import os

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from scirust_b200.models import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.models.infer import InferenceEngine  # noqa: E402
from scirust_b200.ops import _lib, gemm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--quant", default="none", choices=["none", "int8"])
    ap.add_argument("--ttft-iters", type=int, default=5)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (smoke runs)")
    ap.add_argument("--graph", type=int, default=1, help="0: launch every decode step eagerly (for launch lists)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (run under torch.distributed.run)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if a.tp > 1:
        import torch.distributed as dist
        if int(os.environ.get("WORLD_SIZE", "1")) != a.tp:
            raise SystemExit("--tp N needs N ranks: python -m torch.distributed.run --nproc-per-node N ...")
        dist.init_process_group("nccl", device_id=dev)
    cfg = SciAgentConfig.preset(a.model)
    if a.layers:
        cfg.n_layers = a.layers
    model = GQADecoder(cfg, device=dev, seed=7)
    quant = None if a.quant == "none" else "int8"
    if a.tp > 1:
        from scirust_b200.models.infer_tp import TPInferenceEngine
        eng = TPInferenceEngine(model, quant=quant, max_batch=a.batch, max_seq=a.prompt + a.new + 1, page=64,
                                use_graph=bool(a.graph), backend=a.comm)
        n_params = model.num_params()
        del model                      # the shards are copies; free the full weights
        torch.cuda.empty_cache()
    else:
        eng = InferenceEngine(model, quant=quant, max_batch=a.batch, max_seq=a.prompt + a.new + 1, page=64,
                              use_graph=bool(a.graph))
        n_params = model.num_params()
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g).pin_memory()
    # time to first token
    ttft = []
    for i in range(a.ttft_iters + 2):
        for b in range(a.batch):
            if eng.cache.owned[b]:
                eng.cache.release(b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.prefill(prompts)
        first = eng.tokens[:a.batch].cpu()
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            ttft.append(e0.elapsed_time(e1))
    # decode throughput (generate() = prefill + graph-replayed decode)
    l0 = gemm.launch_count
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eng.generate(prompts, 4)            # warm-up: workspaces, graph capture path
    torch.cuda.synchronize()
    e0.record()
    out = eng.generate(prompts, a.new)
    e1.record()
    torch.cuda.synchronize()
    total_ms = e0.elapsed_time(e1)
    p50 = statistics.median(ttft)
    if a.tp > 1:
        t = torch.tensor([p50, total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)          # device times, maximum over ranks
        p50, total_ms = (float(x) for x in t.tolist())
    decode_ms = max(total_ms - p50, 1e-6)
    _lib.check_status(dev)
    if rank == 0:
        print(json.dumps({"metric": "inference", "model": a.model, "layers": cfg.n_layers, "batch": a.batch,
                          "prompt": a.prompt, "new_tokens": a.new, "quant": a.quant, "tp": a.tp,
                          "comm": a.comm if a.tp > 1 else "none", "ttft_p50_ms": p50,
                          "decode_tok_s": a.batch * (a.new - 1) / (decode_ms / 1e3),
                          "decode_ms_per_step": decode_ms / (a.new - 1), "total_ms": total_ms,
                          "params": n_params, "first_tokens": out[:, 0].tolist()[:4]}))
    if a.tp > 1:
        eng.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
