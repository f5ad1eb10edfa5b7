"""Child of tests/test_multigpu.py: 2-rank data-parallel training, fused reducer vs NCCL baseline."""
import os

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)

from scirust_b200.models import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.data_parallel import make_grad_reducer  # noqa: E402
from scirust_b200.train import Trainer, TrainerConfig  # noqa: E402

cfg = SciAgentConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=512, max_seq_len=256,
                     rope_theta=10000.0)


def run(kind):
    model = GQADecoder(cfg, device=dev, seed=3)
    tr = Trainer(model, TrainerConfig(lr=1e-3), grad_reducer=make_grad_reducer(model, dist.group.WORLD, kind=kind))
    g = torch.Generator().manual_seed(10 + rank)
    losses = []
    for _ in range(4):
        tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=g)
        losses.append(float(tr.train_step(tok).item()))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    return losses, model.flat.clone()


l_f, w_f = run("fused")
l_f2, w_f2 = run("fused")
l_n, w_n = run("nccl")
assert torch.equal(w_f, w_f2), "fused data-parallel training is not bitwise repeatable"
# replicas stay identical
ws = [torch.empty_like(w_f) for _ in range(world)]
dist.all_gather(ws, w_f)
assert all(torch.equal(w, ws[0]) for w in ws)
rel = (w_f.float() - w_n.float()).norm() / w_n.float().norm()
assert rel < 2e-3, rel
assert abs(l_f[-1] - l_n[-1]) < 5e-2, (l_f, l_n)
dist.barrier()
if rank == 0:
    print("DP_TRAIN_OK", l_f, l_n, float(rel))
dist.destroy_process_group()
