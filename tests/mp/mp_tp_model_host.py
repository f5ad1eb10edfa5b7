"""Child of tests/test_cpu_parallel.py: the tensor-parallel decoder on the host backend (gloo, CPU tensors) follows the
single-device model: same losses, same updated weights shard for shard, replicated copies identical on every rank."""
import os

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")

from scirust_b200.models import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.models.sciagent_tp import TPDecoder  # noqa: E402
from scirust_b200.parallel.tensor_parallel import TPContext  # noqa: E402
from scirust_b200.train import Trainer, TrainerConfig  # noqa: E402

H = int(os.environ.get("SB_TP_HEADS", "4"))
cfg = SciAgentConfig(vocab_size=512, d_model=16 * H, n_layers=2, n_heads=H, n_kv_heads=int(os.environ.get("SB_TP_KV", "2")),
                     d_ff=128, max_seq_len=128, rope_theta=10000.0)
B, S = max(2, world), 128
g = torch.Generator().manual_seed(7)
batches = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g) for _ in range(3)]
vp = os.environ.get("SB_TP_VOCAB_PARALLEL", "0") == "1"

tp = TPContext(dist.group.WORLD, B * S, cfg.d_model, backend="host")
if vp:
    from scirust_b200.models.sciagent_tp import TPDecoderVocabParallel
    model = TPDecoderVocabParallel(cfg, tp, seed=3)
else:
    model = TPDecoder(cfg, tp, seed=3)
tr = Trainer(model, TrainerConfig(lr=1e-3))
losses = []
for tok in batches:
    l = tr.train_step(tok).detach().clone()
    dist.all_reduce(l)
    losses.append(float(l) / world)
full = GQADecoder(cfg, device="cpu", seed=3)
ft = Trainer(full, TrainerConfig(lr=1e-3))
ref = [float(ft.train_step(t)) for t in batches]
for a, b in zip(losses, ref):
    assert abs(a - b) < 2e-2, (losses, ref)
# the trained shard against the same slice of the trained full model
want = (TPDecoderVocabParallel if vp else TPDecoder)(cfg, tp, seed=99)
want.load_from_full(full)
rel = float((model.flat.float() - want.flat.float()).norm() / want.flat.float().norm())
assert rel < 3e-2, rel
# replicated parameters stay identical on every rank
rs = model.replicated_start
mine = model.flat[rs:].float().clone()
other = mine.clone()
dist.broadcast(other, 0)
assert torch.equal(mine, other), "replicated parameters diverged between ranks"
dist.barrier()
if rank == 0:
    print(f"TP_HOST_OK world={world} kv={cfg.n_kv_heads} vp={int(vp)}", losses, ref, rel)
tp.close()
dist.destroy_process_group()
