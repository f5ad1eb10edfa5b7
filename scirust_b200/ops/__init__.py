"""Native ops. Every function accepts CUDA tensors (hand-written sm_100a kernels) or CPU
tensors (fp32 PyTorch statement of the same arithmetic, used as the oracle)."""
from . import _lib  # noqa: F401
from .gemm import (matmul_nn, matmul_nn_swiglu, matmul_nt, matmul_nt_swiglu_bwd, matmul_tn,  # noqa: F401
                   matmul_tt_a)
from .basic import (rmsnorm_fwd, rmsnorm_bwd, rope_table, rope_, swiglu_fwd, swiglu_bwd, add, embed_fwd,  # noqa: F401
                    embed_bwd, ce_fwd_bwd, ce_loss_only, sumsq, optim_step, multi_cast_to_bf16)
