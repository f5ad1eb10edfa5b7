#!/usr/bin/env python
"""Pipeline parallelism (1F1B) and ring attention on a handful of ranks; runs on CPU ranks (gloo) or on GPUs (NCCL).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        examples/pipeline_and_ring_attention_demo.py [--cuda]

Part 1 trains a small GQA decoder whose layers are split over the ranks (micro-batched 1F1B schedule, per-stage
optimizer, global gradient norm) and writes / reloads a per-stage checkpoint. Part 2 shards one long sequence over the
ranks and computes causal attention with the K/V ring (zigzag layout), comparing with dense attention on rank 0."""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from scirust_b200.models.sciagent import SciAgentConfig  # noqa: E402
from scirust_b200.ops import attention as att  # noqa: E402
from scirust_b200.parallel.context_parallel import ring_attention, shard_sequence  # noqa: E402
from scirust_b200.parallel.pipeline import PipelineModel  # noqa: E402
from scirust_b200.train.trainer import Trainer, TrainerConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--steps", type=int, default=8)
    a = ap.parse_args()
    if a.cuda:
        lr_ = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(lr_)
        dev = torch.device("cuda", lr_)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, W = dist.get_rank(), dist.get_world_size()

    # ---- pipeline-parallel training
    d = 256 if a.cuda else 32
    cfg = SciAgentConfig(vocab_size=512, d_model=d, n_layers=max(4, W), n_heads=4, n_kv_heads=2, d_ff=2 * d,
                         max_seq_len=128, tie_embeddings=False)
    S, micro = (64 if a.cuda else 16), 4
    model = PipelineModel(cfg, device=dev, micro_batches=micro, seed=1)
    trainer = Trainer(model, TrainerConfig(lr=3e-3))
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (2 * micro, S + 1), generator=g)      # the same batch every step
    for step in range(a.steps):
        loss = float(trainer.train_step(data))
        if rank == 0 and step % 2 == 0:
            print(f"[pipeline] step {step}: loss {loss:.4f} (stages {W}, layers {model.lo}..{model.hi - 1} on rank 0)")
    with tempfile.TemporaryDirectory() as tmp:
        shared = [tmp]
        dist.broadcast_object_list(shared, src=0)
        root = model.save_checkpoint(shared[0], a.steps, loss, 3e-3, trainer=trainer)
        meta = model.load_checkpoint(root, trainer=trainer)
        if rank == 0:
            print(f"[pipeline] checkpoint {root.name} reloaded at step {meta['step']}")
        dist.barrier()

    # ---- ring attention over a sequence sharded across the ranks
    B, H, Hkv, dh = 1, 4, 2, 64 if a.cuda else 16
    S_total = (256 if a.cuda else 32) * W
    dt = torch.bfloat16 if a.cuda else torch.float32
    qkv = (torch.randn(B * S_total, (H + 2 * Hkv) * dh, generator=g) * 0.5).to(dt).to(dev)
    local = shard_sequence(qkv, B, S_total, layout="zigzag")
    out = ring_attention(local, B, S_total // W, H, Hkv, dh, causal=True, layout="zigzag")
    ref, _ = att.attention_ref(qkv, B, S_total, H, Hkv, dh, True)
    err = (out.float() - shard_sequence(ref, B, S_total, layout="zigzag")).abs().max().item()
    errs = [None] * W
    dist.all_gather_object(errs, err)
    if rank == 0:
        print(f"[ring attention] {S_total} tokens over {W} ranks (zigzag): max |ring - dense| = {max(errs):.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
