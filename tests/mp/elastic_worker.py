"""Worker of the recovery test (gloo ranks on CPU): data-parallel training of the debug decoder with a checkpoint
every two steps. In attempt 0 rank 1 leaves after step 3, between steps; rank 0 learns it from the heartbeat before
its next collective and exits with the restart code; the supervisor starts both again and they resume from the
latest checkpoint."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def worker(rank, world, attempt, ckpt_dir, port, steps, leave_rank, leave_after):
    from scirust_b200.io import checkpoint as CK
    from scirust_b200.models import GQADecoder, SciAgentConfig
    from scirust_b200.train import Trainer, TrainerConfig
    from scirust_b200.train.elastic import EXIT_PEER_LOST, Heartbeat, PeerLost
    torch.set_num_threads(1)
    store = dist.TCPStore("127.0.0.1", port + attempt, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=60))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    hb = Heartbeat(store, rank, world, timeout_s=20.0, prefix=f"hb{attempt}")
    cfg = SciAgentConfig.debug()
    my_dir = os.path.join(ckpt_dir, f"rank{rank}")
    last = CK.latest_checkpoint(my_dir)
    start = 0
    if last is not None:
        model, meta = CK.load_sciagent_checkpoint(last)
        start = meta["step"]
    else:
        model = GQADecoder(cfg, seed=11)

    def reducer(flat_grad):
        g = flat_grad.float()
        dist.all_reduce(g)                       # two ranks: a + b in either order is the same fp32 value
        flat_grad.copy_((g * (1.0 / world)).to(flat_grad.dtype))
        return 1.0
    tr = Trainer(model, TrainerConfig(lr=1e-2, weight_decay=0.0), grad_reducer=reducer)
    if last is not None:
        CK.load_optimizer_state(model, tr, last)
    losses = []
    for step in range(start, steps):
        try:
            hb.check_peers()
        except PeerLost:
            dist.destroy_process_group()
            return EXIT_PEER_LOST
        g = torch.Generator().manual_seed(1000 * step + rank)
        tok = torch.randint(0, cfg.vocab_size, (2, 17), generator=g)
        try:
            loss = float(tr.train_step(tok).item())
        except RuntimeError:
            # the collective failed under us: the peer went away after our heartbeat check. Same outcome as PeerLost.
            return EXIT_PEER_LOST
        losses.append(loss)
        hb.beat(step + 1)
        if (step + 1) % 2 == 0:
            CK.save_sciagent_checkpoint(model, os.path.join(my_dir, f"step_{step + 1}"), step + 1, loss, 1e-2, trainer=tr)
        if attempt == 0 and rank == leave_rank and step + 1 == leave_after:
            hb.leave("test: rank leaves between steps")
            dist.destroy_process_group()
            return 17
    with open(os.path.join(ckpt_dir, f"final_rank{rank}.txt"), "w") as f:
        f.write(repr(losses[-1]) + "\n" + repr(float(tr.master.double().sum())) + "\n")
    dist.barrier()
    dist.destroy_process_group()
    return 0
