"""Multi-GPU tests (2 ranks as child processes, one GPU each). Skipped with fewer than 2 GPUs.

The fused kernels run on plain peer loads/stores; NVLS is switched off for NCCL in these
children so that a rank leaving between steps cannot disturb a multicast binding."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script: str, nproc: int, port: int, timeout: int = 300, extra_env=None, tag=""):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp", script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    log_dir = os.environ.get("SB_TEST_LOG_DIR")
    if log_dir:
        with open(os.path.join(log_dir, script + tag + ".log"), "w") as f:
            f.write(r.stdout + "\n---- stderr ----\n" + r.stderr)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def test_fused_allreduce_matches_rank_ordered_sum():
    _need(2)
    out = _run("mp_allreduce.py", 2, 29611)
    assert "ALLREDUCE_OK" in out


def test_dp_training_fused_equals_nccl_baseline():
    _need(2)
    out = _run("mp_dp_train.py", 2, 29612)
    assert "DP_TRAIN_OK" in out


def test_tp_fused_layers_match_nccl_baseline():
    _need(2)
    # SB_TP_RS_MIN_GFLOP=0: the tiny test shapes must still take the fused GEMM -> reduce-scatter kernel
    out = _run("mp_tp_layers.py", 2, 29613, extra_env={"SB_TP_RS_MIN_GFLOP": "0"})
    assert "TP_OK" in out


@pytest.mark.parametrize("world,rows", [(2, 256), (2, 768), (2, 200), (4, 256), (4, 768), (8, 256), (8, 768)])
def test_tp_fused_layers_world_and_rows(world, rows):
    """Rows per rank of one and three 256-row blocks (CTA-pair kernels), and off the kernels' row grid, where every
    fused product must refuse cleanly; at every world size the box offers."""
    _need(world)
    out = _run("mp_tp_layers.py", world, 29620 + world, extra_env={"SB_TP_ROWS_PER_RANK": str(rows)},
               tag=f"_w{world}_r{rows}")
    assert f"TP_OK world={world} rows_per_rank={rows}" in out


@pytest.mark.parametrize("world", [4, 8])
def test_fused_allreduce_larger_worlds(world):
    _need(world)
    out = _run("mp_allreduce.py", world, 29630 + world, tag=f"_w{world}")
    assert "ALLREDUCE_OK" in out


def test_tp_decoder_trains_like_single_gpu():
    _need(2)
    out = _run("mp_tp_model.py", 2, 29614, extra_env={"SB_TP_RS_MIN_GFLOP": "0"})
    assert "TP_MODEL_OK" in out


@pytest.mark.parametrize("world,heads,kv,batch", [(2, 4, 1, 2), (4, 4, 2, 4), (8, 8, 2, 8)])
def test_tp_decoder_replicated_kv_heads_and_larger_worlds(world, heads, kv, batch):
    _need(world)
    out = _run("mp_tp_model.py", world, 29640 + world, extra_env={"SB_TP_HEADS": str(heads), "SB_TP_KV": str(kv),
                                                                    "SB_TP_BATCH": str(batch)},
               tag=f"_w{world}_kv{kv}")
    assert f"TP_MODEL_OK world={world} kv={kv}" in out


def test_vocab_parallel_embedding_ce_argmax():
    _need(2)
    out = _run("mp_vocab_parallel.py", 2, 29619)
    assert "VOCAB_PARALLEL_OK" in out


def test_dp_cnn_fused_allreduce_with_overlap():
    _need(2)
    out = _run("mp_dp_cnn.py", 2, 29615)
    assert "DP_CNN_OK" in out


@pytest.mark.parametrize("backend,quant", [("fused", ""), ("nccl", ""), ("fused", "int8")])
def test_tp_inference_matches_single_gpu(backend, quant):
    _need(2)
    out = _run("mp_tp_infer.py", 2, 29616, extra_env={"SB_TEST_DEVICE": "cuda", "SB_TP_BACKEND": backend,
                                                      "SB_TP_QUANT": quant}, tag=f"_{backend}_{quant}")
    assert "TP_INFER_OK" in out and f"backend={backend}" in out


def test_tp_inference_batch16_and_replicated_kv_heads():
    _need(2)
    out = _run("mp_tp_infer.py", 2, 29617, extra_env={"SB_TEST_DEVICE": "cuda", "SB_TP_BATCH": "16", "SB_TP_KV": "1"},
               tag="_b16")
    assert "TP_INFER_OK" in out


@pytest.mark.parametrize("stages,tied", [(2, 0), (4, 1)])
def test_pipeline_parallel_training_over_nccl(stages, tied):
    """1F1B pipeline over NCCL point-to-point transfers: the stages end on the weights of the single-GPU run that
    accumulates the same micro-batches (tests/mp/mp_pipeline.py)."""
    _need(stages)
    out = _run("mp_pipeline.py", stages, 29680 + stages, tag=f"_p{stages}",
               extra_env={"SB_PP_CUDA": "1", "SB_PP_TIED": str(tied), "SB_PP_MICRO": "4"})
    assert "PIPELINE_OK" in out


@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_over_nccl(world):
    """Context parallelism on the flash kernels: every hop is one attention_fwd / attention_bwd launch on the
    visiting K/V shard, merged by log-sum-exp; equals dense attention over the whole sequence."""
    _need(world)
    out = _run("mp_ring_attention.py", world, 29690 + world, tag=f"_w{world}", extra_env={"SB_CP_CUDA": "1"})
    assert "RING_ATTENTION_OK" in out
