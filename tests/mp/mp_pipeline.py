"""Pipeline-parallel training on P ranks (gloo on CPU, NCCL when SB_PP_CUDA=1): after three optimizer steps every stage
holds the weights of the single-process run that accumulates the same micro-batches."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from scirust_b200.models.sciagent import GQADecoder, SciAgentConfig  # noqa: E402
from scirust_b200.parallel.pipeline import InterleavedPipelineModel, PipelineModel, split_layers  # noqa: E402
from scirust_b200.train.trainer import Trainer, TrainerConfig  # noqa: E402


def _close(a, b, lr=5e-3, steps=3):
    """Tied embeddings make the two runs differ in the last bits of one gradient; under Adam an element whose gradient
    is near zero may then step the other way, so: nothing farther apart than the optimizer can move an element in the
    run, and all but a small fraction within a rounding of each other."""
    d = (a.float() - b.float()).abs()
    far = int((d > 2e-3 + 2.0 ** -7 * b.float().abs()).sum())
    return bool(d.max() <= 2 * lr * steps + 1e-3) and far <= max(2, int(0.02 * d.numel()))


def main():
    use_cuda = os.environ.get("SB_PP_CUDA") == "1"
    rank = int(os.environ["RANK"])
    if use_cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    P = dist.get_world_size()
    tied = os.environ.get("SB_PP_TIED", "0") == "1"
    M = int(os.environ.get("SB_PP_MICRO", "4"))
    V = int(os.environ.get("SB_PP_VIRTUAL", "1"))
    d = 256 if use_cuda else 32
    cfg = SciAgentConfig(vocab_size=512 if use_cuda else 96, d_model=d, n_layers=5 if V == 1 else P * V + 1, n_heads=4, n_kv_heads=2,
                         d_ff=2 * d, max_seq_len=128, tie_embeddings=tied)
    S = 64 if use_cuda else 16
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (3, 2 * M, S + 1), generator=g)
    full = GQADecoder(cfg, device=dev, seed=11)
    make = (lambda **kw: PipelineModel(cfg, device=dev, micro_batches=M, **kw)) if V == 1 else \
        (lambda **kw: InterleavedPipelineModel(cfg, device=dev, micro_batches=M, virtual_stages=V, **kw))
    pm = make()
    pm.load_from_full(full)
    # clipping stays inactive: the pipeline adds the squared norm stage by stage, another association than one pass
    # over the whole buffer, and an active clip factor would differ in its last bit
    tcfg = TrainerConfig(lr=5e-3, max_grad_norm=1e6)
    tr = Trainer(pm, tcfg)
    pp_losses = [float(tr.train_step(t)) for t in data]
    pp_norm = tr.grad_norm()

    # single process, same micro-batches accumulated in the same order
    class Accum:
        """The complete model behind the Trainer interface, fed micro-batch by micro-batch."""

        def __init__(self, m):
            self.m, self.flat, self.flat_grad, self.decay_end = m, m.flat, m.flat_grad, m.decay_end

        def zero_grad_flags(self):
            self.m.zero_grad_flags()

        def __call__(self, inp, tgt):
            mb = inp.shape[0] // M
            tot = 0.0
            for i in range(M):
                l = self.m(inp[i * mb:(i + 1) * mb], tgt[i * mb:(i + 1) * mb])
                (l * (1.0 / M)).backward()
                tot = tot + l.detach().float()
            return (tot / M).requires_grad_()
    ref = Trainer(Accum(full), tcfg)
    ref_losses = [float(ref.train_step(t)) for t in data]
    # tied embeddings: the two end stages round their halves of the table's gradient to bf16 before they are summed,
    # the single process accumulates the second half onto the rounded first, so that run agrees closely, not bitwise
    ltol = 1e-4 if tied else 1e-6
    assert all(abs(a - b) <= ltol * max(1.0, abs(b)) for a, b in zip(pp_losses, ref_losses)), (pp_losses, ref_losses)
    # the deeper model of the interleaved runs amplifies the tied table's rounding difference more by the third step
    # (the plain and the interleaved pipeline still agree with each other to the last bit)
    ntol = (5e-3 if V == 1 else 2e-2) if tied else 1e-4
    assert abs(pp_norm - ref.grad_norm()) <= ntol * max(1.0, ref.grad_norm()), (pp_norm, ref.grad_norm())
    mine = list(range(*split_layers(cfg.n_layers, P)[rank])) if V == 1 else [i for lo, hi, _ in pm.chunks for i in range(lo, hi)]
    local = (lambda i: pm.stage.layers[i - mine[0]]) if V == 1 else pm.local_layer
    assert len(mine) == len(pm.stage.layers)
    for i in mine:
        for name in ("rms_attn", "wqkv", "wo", "rms_ffn", "wgu", "wd"):
            a, b = getattr(local(i), name), getattr(full.layers[i], name)
            same = _close(a, b) if tied else torch.equal(a, b)
            assert same, f"stage {rank}: layer {i} {name} differs by {(a.float() - b.float()).abs().max()}"
    close = _close if tied else torch.equal
    if rank == 0:
        assert close(pm.stage.embed, full.embed)
    if rank == P - 1:
        assert close(pm.stage.rms_final, full.rms_final)
        assert close(pm.stage.head_weight(), full.head_weight())
    # checkpoint / resume: two steps, save, a fresh stage + trainer resumes and takes the third step; its weights are
    # the bits of the run that took three steps without stopping (pm above)
    ckpt = os.environ.get("SB_PP_CKPT")
    if ckpt:
        full2 = GQADecoder(cfg, device=dev, seed=11)
        a = make()
        a.load_from_full(full2)
        ta = Trainer(a, tcfg)
        for t in data[:2]:
            last = ta.train_step(t)
        root = a.save_checkpoint(ckpt, 2, float(last), tcfg.lr, trainer=ta)
        assert PipelineModel.latest(ckpt) == root
        b = make(seed=99)                                                # other initial weights: everything must come from disk
        tb = Trainer(b, tcfg)
        assert b.load_checkpoint(root, trainer=tb)["step"] == 2 and tb.step == 2
        tb.train_step(data[2])
        assert torch.equal(b.stage.flat, pm.stage.flat), "resumed pipeline stage differs from the uninterrupted run"
    dist.barrier()
    if rank == 0:
        print(f"PIPELINE_OK stages={P} virtual={V} micro={M} tied={tied} loss={pp_losses[-1]:.4f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
