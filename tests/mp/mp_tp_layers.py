"""Child of tests/test_multigpu.py: fused all-gather->GEMM / GEMM->reduce-scatter products against
the NCCL + library-GEMM baseline and an fp32 reference; bitwise repeatability."""
import os

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)

from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.tensor_parallel import TPContext  # noqa: E402

BF = torch.bfloat16
# tokens, model dim, column shard, row shard; rows per rank from the environment (a multiple of 256 runs on the
# CTA-pair kernels, anything else on the single-CTA distributed kernel)
ROWS = int(os.environ.get("SB_TP_ROWS_PER_RANK", "512"))
T, d, Nr, Kr = ROWS * world, 512, 384, 256
Tl = T // world
N_ODD = 320      # an output width that ends inside a 64-column store slab and a 256-column tile


def rnd(shape, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=dev) * 0.3).to(BF)


fused = TPContext(dist.group.WORLD, T, d, sym_bytes=64 << 20, backend="fused")
base = TPContext(dist.group.WORLD, T, d, backend="nccl")

# identical "global" tensors on every rank (same seeds), sharded by rank where needed
x_full = rnd((T, d), 1)
x_shard = fused.buffer("x", (Tl, d)); x_shard.copy_(x_full[rank * Tl:(rank + 1) * Tl])
w_col = rnd((d, Nr), 10 + rank)          # column-parallel weight shard [in, out_r]
w_row = rnd((Kr, d), 20 + rank)          # row-parallel weight shard [in_r, out]
a_loc = rnd((T, Kr), 30 + rank)          # local activation with all tokens (row-parallel input)
dy_loc = rnd((T, Nr), 40 + rank)         # local gradient with all tokens (column-parallel output grad)
dy_full = rnd((T, d), 2)
dy_shard = fused.buffer("dy", (Tl, d)); dy_shard.copy_(dy_full[rank * Tl:(rank + 1) * Tl])
res = rnd((Tl, d), 50 + rank)
w_row_odd = rnd((Kr, N_ODD), 60 + rank)  # row-parallel weight with a ragged output width
x_odd_full = rnd((T, N_ODD), 3)          # gathered operand with a ragged contraction width
x_odd = fused.buffer("x_odd", (Tl, N_ODD)); x_odd.copy_(x_odd_full[rank * Tl:(rank + 1) * Tl])
w_col_odd = rnd((N_ODD, Nr), 70 + rank)


def close(a, b, what):
    err = (a.float() - b.float()).abs().max().item()
    lim = 3e-2 * max(1.0, b.float().abs().max().item())
    assert err <= lim, f"{what}: {err} > {lim}"


def sync():
    torch.cuda.synchronize()
    _lib.check_status(dev)


if ROWS % 128:
    # rows per rank off the kernels' 128-row grid: every fused product must refuse on the host (a typed error, the
    # same on all ranks) instead of computing something
    refused = 0
    for call in (lambda: fused.ag_matmul_nn(x_shard, w_col), lambda: fused.matmul_nn_rs(a_loc, w_row),
                 lambda: fused.matmul_nt_rs(dy_loc, w_col)):
        try:
            call()
        except (_lib.NativeError, ValueError):
            refused += 1
    sync()
    assert refused == 3, f"only {refused} of 3 off-grid products were refused"
    dist.barrier()
    if rank == 0:
        print(f"TP_OK world={world} rows_per_rank={ROWS} (refused)")
    fused.close()
    dist.destroy_process_group()
    raise SystemExit(0)


for rep in range(2):
    # all-gather -> GEMM (forward of column-parallel, and input-gradient of row-parallel)
    y1 = fused.ag_matmul_nn(x_shard, w_col); sync()
    close(y1, x_full.float() @ w_col.float(), "ag_matmul_nn")
    close(y1, base.ag_matmul_nn(x_shard, w_col), "ag_matmul_nn vs nccl")
    y2 = fused.ag_matmul_nt(dy_shard, w_row); sync()
    close(y2, dy_full.float() @ w_row.float().t(), "ag_matmul_nt")

    # GEMM -> reduce-scatter (forward of row-parallel with fused residual, input-gradient of column-parallel)
    parts = [torch.empty((T, d), dtype=torch.float32, device=dev) for _ in range(world)]
    dist.all_gather(parts, (a_loc.float() @ w_row.float()))
    ref = sum(p[rank * Tl:(rank + 1) * Tl] for p in parts) + res.float()
    y3 = fused.matmul_nn_rs(a_loc, w_row, residual_shard=res); sync()
    close(y3, ref, "matmul_nn_rs")
    close(y3, base.matmul_nn_rs(a_loc, w_row, residual_shard=res), "matmul_nn_rs vs nccl")
    dist.all_gather(parts, (dy_loc.float() @ w_col.float().t()))
    ref = sum(p[rank * Tl:(rank + 1) * Tl] for p in parts)
    y4 = fused.matmul_nt_rs(dy_loc, w_col); sync()
    close(y4, ref, "matmul_nt_rs")

    # ragged widths: output columns / contraction length that are not multiples of the tile sizes
    parts_o = [torch.empty((T, N_ODD), dtype=torch.float32, device=dev) for _ in range(world)]
    dist.all_gather(parts_o, (a_loc.float() @ w_row_odd.float()))
    ref = sum(p[rank * Tl:(rank + 1) * Tl] for p in parts_o)
    y5 = fused.matmul_nn_rs(a_loc, w_row_odd); sync()
    close(y5, ref, "matmul_nn_rs ragged N")
    y6 = fused.ag_matmul_nn(x_odd, w_col_odd); sync()
    close(y6, x_odd_full.float() @ w_col_odd.float(), "ag_matmul_nn ragged K")

    # weight gradients with one operand gathered along the contraction (token) dimension
    g1 = fused.ag_matmul_tn(x_shard, dy_loc); sync()
    close(g1, x_full.float().t() @ dy_loc.float(), "ag_matmul_tn")
    g2 = fused.matmul_tn_ag(a_loc, dy_shard); sync()
    close(g2, a_loc.float().t() @ dy_full.float(), "matmul_tn_ag")
    if rep == 0:
        first = [t.clone() for t in (y1, y2, y3, y4, y5, y6, g1, g2)]
    else:
        for a, b in zip(first, (y1, y2, y3, y4, y5, y6, g1, g2)):
            assert torch.equal(a, b), "fused tensor-parallel products are not bitwise repeatable"

# two fused products in flight on two streams (each with its own context: flag slots, staging and landing buffers
# are per context), interleaved with each other on the GPU
other = TPContext(dist.group.WORLD, T, d, sym_bytes=8 << 20, backend="fused")
x_b = other.buffer("x", (Tl, d)); x_b.copy_(x_shard)
side = torch.cuda.Stream()
side.wait_stream(torch.cuda.current_stream())
for _ in range(3):
    ya = fused.matmul_nn_rs(a_loc, w_row, residual_shard=res)
    with torch.cuda.stream(side):
        yb = other.ag_matmul_nn(x_b, w_col)
torch.cuda.current_stream().wait_stream(side)
sync()
assert torch.equal(ya, first[2]) and torch.equal(yb, first[0]), "concurrent fused products disturbed one another"
other.close()

dist.barrier()
if rank == 0:
    print(f"TP_OK world={world} rows_per_rank={ROWS}")
fused.close()
dist.destroy_process_group()
