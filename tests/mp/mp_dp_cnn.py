"""Child of tests/test_multigpu.py: data-parallel CNN training on the fused gradient all-reduce with
overlap; replicas stay bitwise identical and track the NCCL baseline."""
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)

from scirust_b200.models.cnn import MnistCNN  # noqa: E402
from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.ddp import FlatDataParallel  # noqa: E402


def run(comm):
    model = MnistCNN(seed=1).to(dev)
    dp = FlatDataParallel(model, dist.group.WORLD, optimizer="adam", lr=1e-3, comm=comm, bucket_elems=1 << 18)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(5):
        x = torch.rand(64, 784, generator=g).to(dev)
        y = torch.randint(0, 10, (64,), generator=g).to(dev)
        loss = F.cross_entropy(dp(x), y)
        loss.backward()
        dp.step()
        losses.append(float(loss.detach()))
    torch.cuda.synchronize()
    _lib.check_status(dev)
    w = dp.master.clone()
    dp.close()
    return losses, w


lf, wf = run("fused")
lf2, wf2 = run("fused")
ln, wn = run("nccl")
assert torch.equal(wf, wf2), "fused data-parallel CNN training is not bitwise repeatable"
ws = [torch.empty_like(wf) for _ in range(world)]
dist.all_gather(ws, wf)
assert all(torch.equal(w, ws[0]) for w in ws), "replicas diverged"
rel = (wf - wn).norm() / wn.norm()
assert rel < 5e-2, rel
dist.barrier()
if rank == 0:
    print("DP_CNN_OK", lf, ln, float(rel))
dist.destroy_process_group()
