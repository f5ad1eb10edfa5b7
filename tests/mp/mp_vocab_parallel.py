"""Vocabulary-parallel embedding / cross-entropy / arg-max against the single-device ops (gloo or NCCL ranks)."""
import os
import sys

import torch
import torch.distributed as dist

cpu = os.environ.get("SB_TEST_DEVICE", "cuda") == "cpu"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
if cpu:
    dev = torch.device("cpu")
    dist.init_process_group("gloo")
else:
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)

from scirust_b200.ops import basic  # noqa: E402
from scirust_b200.parallel import vocab_parallel as VP  # noqa: E402

dt = torch.float32 if cpu else torch.bfloat16
V, d, n = 512 * world, 64, 300
g = torch.Generator().manual_seed(7)
table = (torch.randn(V, d, generator=g) * 0.5).to(dt).to(dev)
h = (torch.randn(n, d, generator=g) * 0.5).to(dt).to(dev)
tok = torch.randint(0, V, (n,), generator=g).to(dev)
tgt = torch.randint(0, V, (n,), generator=g)
tgt[::17] = -1
tgt = tgt.to(dev)
v0, per = VP.shard_range(V, rank, world)
shard = table[v0:v0 + per].contiguous()

# embedding forward / backward
emb = VP.VocabParallelEmbedding(shard, V)
x = emb.forward(tok)
assert torch.equal(x, basic.embed_fwd(table, tok)), "embedding forward"
dy = (torch.randn(n, d, generator=g) * 0.1).to(dt).to(dev)
dsh = torch.zeros_like(shard)
emb.backward(dy, tok, dsh, accumulate=False)
dfull = torch.zeros_like(table)
basic.embed_bwd(dy, tok, dfull, accumulate=False)
assert torch.allclose(dsh.float(), dfull[v0:v0 + per].float(), atol=1e-6), "embedding backward"

# cross-entropy
logits_full = (h.float() @ table.float().t()).to(dt)
local = logits_full[:, v0:v0 + per].contiguous()
loss, dl = VP.vocab_parallel_ce(local.clone(), tgt, v0, 1.0 / n)
lf = logits_full.float()
ref_lse = torch.logsumexp(lf, -1)
ref_loss = torch.where(tgt < 0, torch.zeros_like(ref_lse), ref_lse - lf.gather(1, tgt.clamp(min=0)[:, None])[:, 0])
assert (loss - ref_loss).abs().max().item() < (1e-4 if cpu else 2e-2), (loss - ref_loss).abs().max().item()
p = torch.softmax(lf, -1)
p[torch.arange(n, device=dev), tgt.clamp(min=0)] -= 1
p = p / n
p[tgt < 0] = 0
err = (dl.float() - p[:, v0:v0 + per]).abs().max().item()
assert err < (1e-6 if cpu else 1e-4), err
loss2, dl2 = VP.vocab_parallel_ce(local.clone(), tgt, v0, 1.0 / n)
assert torch.equal(loss, loss2) and torch.equal(dl, dl2), "repeatability"
gl = [torch.empty_like(loss) for _ in range(world)]
dist.all_gather(gl, loss)
assert all(torch.equal(gl[0], t) for t in gl), "every rank sees the same loss"

# arg-max, ties included
local2 = local.clone()
local2[5, :] = 0
am = VP.vocab_parallel_argmax(local2, v0)
full2 = logits_full.clone()
full2[5, :] = 0
ref_am = full2.float().argmax(-1)
keep = torch.ones(n, dtype=torch.bool, device=dev)
keep[5] = False
assert torch.equal(am[keep], ref_am[keep]), "arg-max"
assert am[5].item() == 0, "a tie goes to the smallest id"
if not cpu:
    from scirust_b200.ops import _lib
    _lib.check_status(dev)
dist.barrier()
if rank == 0:
    print("VOCAB_PARALLEL_OK")
dist.destroy_process_group()
