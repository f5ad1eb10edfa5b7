"""Ring attention on W ranks (gloo on CPU; NCCL with SB_CP_CUDA=1): output and qkv gradient of every rank's slice equal
the slice of dense attention over the whole sequence."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from scirust_b200.ops import attention as att  # noqa: E402
from scirust_b200.parallel.context_parallel import ring_attention, shard_sequence  # noqa: E402


def main():
    use_cuda = os.environ.get("SB_CP_CUDA") == "1"
    if use_cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    rank, W = dist.get_rank(), dist.get_world_size()
    B, H, Hkv, dh = 2, 4, 2, 64 if use_cuda else 16
    S = (256 if use_cuda else 24) * W
    dt = torch.bfloat16 if use_cuda else torch.float32
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(B * S, (H + 2 * Hkv) * dh, generator=g) * 0.5).to(dt).to(dev)
    do = (torch.randn(B * S, H * dh, generator=g) * 0.5).to(dt).to(dev)
    from scirust_b200.parallel.context_parallel import visible_pairs
    assert len(set(visible_pairs(W, "zigzag"))) == 1 and visible_pairs(W, "contiguous")[-1] == W * visible_pairs(W, "contiguous")[0]
    for layout in ("contiguous", "zigzag"):
        for causal in (True, False):
            ref_o, _ = att.attention_ref(qkv, B, S, H, Hkv, dh, causal)
            ref_g = att.attention_bwd_ref(qkv, do, B, S, H, Hkv, dh, causal)
            local = shard_sequence(qkv, B, S, layout=layout).requires_grad_()
            out = ring_attention(local, B, S // W, H, Hkv, dh, causal=causal, layout=layout)
            out.backward(shard_sequence(do, B, S, layout=layout))
            tol = 3e-2 if use_cuda else 2e-5
            eo = (out.float() - shard_sequence(ref_o, B, S, layout=layout)).abs().max().item()
            eg = (local.grad.float() - shard_sequence(ref_g, B, S, layout=layout)).abs().max().item()
            assert eo <= tol and eg <= tol * 4, (rank, layout, causal, eo, eg)
            # repeatable bit for bit
            local2 = shard_sequence(qkv, B, S, layout=layout).requires_grad_()
            out2 = ring_attention(local2, B, S // W, H, Hkv, dh, causal=causal, layout=layout)
            out2.backward(shard_sequence(do, B, S, layout=layout))
            assert torch.equal(out, out2) and torch.equal(local.grad, local2.grad)
    dist.barrier()
    if rank == 0:
        print(f"RING_ATTENTION_OK world={W} S={S}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
