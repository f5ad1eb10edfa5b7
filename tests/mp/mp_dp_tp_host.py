"""Child of tests/test_cpu_parallel.py: data parallel x tensor parallel on a 2-D mesh of gloo ranks. Tensor-parallel
groups hold one replica each and see the same batch; replicas see different batches; gradients are summed over the
data-parallel axis. The losses and the trained shards follow a single-device model trained on the concatenated batch."""
import os

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")

from scirust_b200.models import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.models.sciagent_tp import TPDecoder, TPDecoderVocabParallel  # noqa: E402
from scirust_b200.parallel import make_grad_reducer  # noqa: E402
from scirust_b200.parallel.mesh import DeviceMesh  # noqa: E402
from scirust_b200.parallel.tensor_parallel import TPContext  # noqa: E402
from scirust_b200.train import Trainer, TrainerConfig  # noqa: E402

dp, tpw = int(os.environ.get("SB_DP", "2")), int(os.environ.get("SB_TP", "2"))
mesh = DeviceMesh(("dp", "tp"), (dp, tpw))
groups = mesh.process_groups()
me = mesh.coords(rank)
assert dist.get_world_size(groups["tp"]) == tpw and dist.get_world_size(groups["dp"]) == dp
assert mesh.group_ranks("tp", rank) == list(range(me["dp"] * tpw, (me["dp"] + 1) * tpw))

cfg = SciAgentConfig(vocab_size=512, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=128, max_seq_len=128, rope_theta=10000.0)
B, S = tpw, 128                                                       # per replica
g = torch.Generator().manual_seed(11)
steps = [torch.randint(0, cfg.vocab_size, (dp * B, S + 1), generator=g) for _ in range(3)]
vp = os.environ.get("SB_TP_VOCAB_PARALLEL", "0") == "1"

tp = TPContext(groups["tp"], B * S, cfg.d_model, backend="host")
cls = TPDecoderVocabParallel if vp else TPDecoder
model = cls(cfg, tp, seed=5)
tr = Trainer(model, TrainerConfig(lr=1e-3), grad_reducer=make_grad_reducer(model, groups["dp"], kind="nccl"))
losses = []
for tok in steps:
    mine = tok[me["dp"] * B:(me["dp"] + 1) * B]
    l = tr.train_step(mine).detach().clone()
    dist.all_reduce(l)
    losses.append(float(l) / world)
full = GQADecoder(cfg, device="cpu", seed=5)
ft = Trainer(full, TrainerConfig(lr=1e-3))
ref = [float(ft.train_step(t)) for t in steps]
for a, b in zip(losses, ref):
    assert abs(a - b) < 2e-2, (losses, ref)
want = cls(cfg, tp, seed=99)
want.load_from_full(full)
rel = float((model.flat.float() - want.flat.float()).norm() / want.flat.float().norm())
assert rel < 3e-2, rel
# replicas stay identical: the same tensor-parallel shard on every data-parallel rank
mine = model.flat.float().clone()
other = mine.clone()
dist.broadcast(other, mesh.group_ranks("dp", rank)[0], group=groups["dp"])
assert torch.equal(mine, other), "data-parallel replicas diverged"
dist.barrier()
if rank == 0:
    print(f"DP_TP_HOST_OK dp={dp} tp={tpw} vp={int(vp)}", losses, ref, rel)
tp.close()
dist.destroy_process_group()
