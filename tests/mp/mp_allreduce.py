"""Child of tests/test_multigpu.py: fused all-reduce vs a rank-ordered fp32 sum, bitwise repeatable."""
import os
import sys

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)

from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.fused_allreduce import FusedAllReduce  # noqa: E402
from scirust_b200.parallel.symm import SymmetricRegion  # noqa: E402

n = 8 * 1000 * 125 + 8 * 3  # not divisible by world*8
region = SymmetricRegion(dist.group.WORLD, n * 2 * 2 + 8192)
src = region.tensor((n,), torch.bfloat16)
dst = region.tensor((n,), torch.bfloat16)
ar = FusedAllReduce(region, src, dst, n_ctas=16)

results = []
for it in range(3):
    g = torch.Generator(device=dev).manual_seed(100 * it + rank)
    src.copy_(torch.randn(n, generator=g, device=dev).to(torch.bfloat16))
    ar.reduce(0, n, 1.0 / world, ar.next_epoch(), lean=(it == 1))      # the small CTA shape gives the same bits
    torch.cuda.synchronize()
    _lib.check_status(dev)
    # oracle: gather every rank's input, add in rank order in fp32, scale, round once
    parts = [torch.empty_like(src) for _ in range(world)]
    dist.all_gather(parts, src.clone())
    acc = torch.zeros(n, dtype=torch.float32, device=dev)
    for p in parts:
        acc += p.float()
    ref = (acc * (1.0 / world)).to(torch.bfloat16)
    assert torch.equal(dst, ref), (it, (dst.float() - ref.float()).abs().max().item())
    results.append(dst.clone())
# all ranks hold identical bits
chk = [torch.empty_like(dst) for _ in range(world)]
dist.all_gather(chk, dst.clone())
assert all(torch.equal(c, chk[0]) for c in chk)

# a wait that nothing satisfies returns a status instead of hanging
flags = torch.zeros(16, dtype=torch.int32, device=dev)
lib = _lib.cuda()
st = _lib.status_word(dev)
assert lib.sb_wait_probe(flags.data_ptr(), 2, 7, 200, st.data_ptr(), _lib.stream()) == 0
torch.cuda.synchronize()
assert int(st.item()) == 5
st.zero_()

dist.barrier()
if rank == 0:
    print("ALLREDUCE_OK")
region.close()
dist.destroy_process_group()
