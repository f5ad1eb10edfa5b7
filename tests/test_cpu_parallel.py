"""Host-side collectives (threads and TCP as ranks), data-parallel determinism, logical sharding,
gloo process groups; failures are injected on the host."""
import os
import socket
import subprocess
import sys
import threading

import numpy as np
import pytest
import torch

from scirust_b200.nn.rng import Philox4x32
from scirust_b200.parallel import host_collectives as HC
from scirust_b200.parallel.mesh import DeviceMesh, PartitionSpec, ShardingError, plan_sharding, shard_map

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(world, n, seed=7):
    return [Philox4x32(seed).fill_f32(r, 0, n) * np.float32(10 ** (r % 5 - 2)) for r in range(world)]


def test_thread_allreduce_is_rank_ordered_mean():
    xs = _inputs(4, 257)

    def fn(ctx):
        out = ctx.all_reduce("g", xs[ctx.rank])
        b = ctx.broadcast("w", xs[0] if ctx.rank == 0 else None)
        ctx.barrier()
        return out, b
    res = HC.run_ranks(4, fn)
    acc = np.zeros(257, np.float32)
    for x in xs:
        acc = (acc + x).astype(np.float32)
    want = (acc * np.float32(0.25)).astype(np.float32)
    for out, b in res:
        assert np.array_equal(out, want) and np.array_equal(b, xs[0])


def test_thread_allreduce_mismatch_is_an_error_on_every_rank():
    def fn(ctx):
        return ctx.all_reduce("g", np.zeros(3 if ctx.rank else 4, np.float32))
    with pytest.raises(HC.CollectiveError):
        HC.run_ranks(3, fn)

    def fn2(ctx):
        return ctx.all_reduce_dict({"a": np.zeros(2), ("b" if ctx.rank else "c"): np.zeros(2)})
    with pytest.raises(HC.CollectiveError):
        HC.run_ranks(2, fn2)


@pytest.mark.parametrize("world", [1, 2, 5, 8])
def test_tree_allreduce_jitter_never_changes_bits(world):
    xs = _inputs(world, 129)
    base = HC.tree_all_reduce(xs)
    for seed in (1, 2, 3):
        again = HC.tree_all_reduce(xs, jitter_seed=seed)
        assert all(np.array_equal(a, base[0]) for a in again)
    exact = HC.tree_all_reduce(xs, combine=HC.ExactSum, jitter_seed=4)
    import math
    want = np.array([np.float32(math.fsum(float(x[i]) for x in xs)) for i in range(129)], np.float32)
    assert np.array_equal(exact[0], want)        # topology-independent, correctly rounded


def _free_ports(n):
    socks = [socket.socket() for _ in range(n)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


def test_tcp_tree_allreduce_matches_in_process_engine():
    world = 5
    xs = _inputs(world, 64)
    addrs = [("127.0.0.1", p) for p in _free_ports(world)]
    out, errs = [None] * world, []

    def work(r):
        try:
            out[r] = HC.tcp_tree_all_reduce_rank(r, world, addrs, xs[r], timeout=20)
        except Exception as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
    ref = HC.tree_all_reduce(xs)[0]
    assert all(np.array_equal(o, ref) for o in out)


def test_tcp_frames_reject_unexpected_rank_and_oversize():
    a, b = socket.socketpair()
    HC.send_frame(a, 9, b"abc")
    with pytest.raises(HC.CollectiveError):
        HC.recv_frame(b, {1, 2})
    a.sendall((1).to_bytes(4, "little") + (HC.MAX_FRAME + 1).to_bytes(8, "little"))
    with pytest.raises(HC.CollectiveError):
        HC.recv_frame(b, {1})
    a.close()
    with pytest.raises(HC.CollectiveError):
        HC.recv_frame(b, {1})                      # peer went away mid-frame
    b.close()


def test_tcp_rank_that_never_joins_times_out_cleanly():
    addrs = [("127.0.0.1", p) for p in _free_ports(3)]
    with pytest.raises((HC.CollectiveError, OSError)):
        HC.tcp_tree_all_reduce_rank(0, 3, addrs, np.ones(4, np.float32), timeout=0.5)   # children never connect


def test_data_parallel_update_is_identical_for_any_worker_count_and_threading():
    rs = np.random.RandomState(0)
    x, y = rs.randn(64, 6).astype(np.float32), rs.randn(64, 1).astype(np.float32)

    def grad_fn(params, xb, yb):
        w = params[0]
        err = xb @ w - yb
        return float((err ** 2).mean()), [(2.0 / len(xb)) * (xb.T @ err)]

    def upd(params, grads):
        params[0] -= np.float32(0.05) * grads[0]
    finals = {}
    for threaded in (False, True):
        p = [np.zeros((6, 1), np.float32)]
        t = HC.DataParallelTrainer(4, grad_fn, upd)
        for _ in range(5):
            (t.train_batch_threaded if threaded else t.train_batch)(p, x, y)
        finals[threaded] = p[0].copy()
    assert np.array_equal(finals[False], finals[True])


def test_mesh_and_shard_map():
    mesh = DeviceMesh(("dp", "tp"), (2, 2))
    assert mesh.coords(3) == {"dp": 1, "tp": 1} and mesh.group_ranks("tp", 2) == [2, 3]
    x, w = torch.randn(8, 6), torch.randn(6, 4)
    y = shard_map(lambda a, b: a @ b, mesh, (PartitionSpec("dp", None), PartitionSpec(None, "tp")),
                  PartitionSpec("dp", "tp"), x, w)
    assert torch.allclose(y, x @ w, atol=1e-6)
    z = shard_map(lambda a: a.sum(0, keepdim=True) * 0 + 1, mesh, (PartitionSpec(None, None),), PartitionSpec(None, None), x)
    assert z.shape == (1, 6)
    with pytest.raises(ShardingError):
        plan_sharding((7, 4), PartitionSpec("dp", None), mesh)
    with pytest.raises(ShardingError):
        shard_map(lambda a: a[:1] , mesh, (PartitionSpec("dp", None),), PartitionSpec(None, None), x)


def test_gloo_ranks_rank_that_raises_fails_the_job():
    code = (
        "import os, sys, datetime, torch, torch.distributed as dist\n"
        "dist.init_process_group('gloo', timeout=datetime.timedelta(seconds=5))\n"
        "r = dist.get_rank()\n"
        "t = torch.ones(4) * (r + 1)\n"
        "dist.all_reduce(t)\n"
        "assert t[0] == 3\n"
        "if os.environ.get('FAIL_RANK') == str(r):\n"
        "    raise SystemExit(3)          # leaves between steps, nothing in flight\n"
        "try:\n"
        "    dist.all_reduce(t)\n"
        "    print('SECOND_OK')\n"
        "except Exception as e:\n"
        "    print('PEER_LOST', type(e).__name__)\n"
        "    sys.exit(0)\n")
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
            "127.0.0.1", "--master-port", "29631", "-c" if False else "--no-python", sys.executable, "-c", code]
    ok = subprocess.run(base, capture_output=True, text=True, timeout=120, env=dict(os.environ, PYTHONPATH=ROOT))
    assert ok.returncode == 0 and ok.stdout.count("SECOND_OK") == 2, ok.stdout + ok.stderr
    bad = subprocess.run(base, capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, PYTHONPATH=ROOT, FAIL_RANK="1"))
    assert bad.returncode != 0
    assert "PEER_LOST" in bad.stdout or "SECOND_OK" not in bad.stdout


@pytest.mark.parametrize("world,kv", [(2, 4), (4, 1)])
def test_tp_inference_engine_on_gloo_ranks(world, kv):
    """Tensor-parallel sharding, row-parallel reductions and the vocabulary-parallel head, on CPU ranks."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29650 + world), os.path.join(ROOT, "tests", "mp", "mp_tp_infer.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_TP_KV=str(kv), SB_TEST_DEVICE="cpu"))
    assert r.returncode == 0 and "TP_INFER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("world", [2, 4])
def test_vocab_parallel_embedding_ce_argmax_on_gloo_ranks(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29660 + world), os.path.join(ROOT, "tests", "mp", "mp_vocab_parallel.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_TEST_DEVICE="cpu"))
    assert r.returncode == 0 and "VOCAB_PARALLEL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("stages,tied,micro", [(2, 0, 4), (3, 1, 2)])
def test_pipeline_parallel_1f1b_equals_single_process_accumulation_on_gloo_ranks(stages, tied, micro, tmp_path):
    """Layers split over 2 / 3 stages, 1F1B over the micro-batches, per-stage optimizer with a global gradient norm:
    three steps end on the weights of the single-process run that accumulates the same micro-batches; a run that is
    checkpointed after two steps and resumed by fresh stages ends on the same bits."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={stages}", "--master-addr",
           "127.0.0.1", "--master-port", str(29670 + stages), os.path.join(ROOT, "tests", "mp", "mp_pipeline.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_PP_TIED=str(tied), SB_PP_MICRO=str(micro),
                                SB_PP_CKPT=str(tmp_path / "pp")))
    assert r.returncode == 0 and "PIPELINE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("stages,virtual,tied,micro", [(2, 2, 0, 4), (3, 2, 1, 3), (2, 3, 0, 2)])
def test_interleaved_pipeline_equals_single_process_accumulation_on_gloo_ranks(stages, virtual, tied, micro, tmp_path):
    """Virtual stages: every rank owns several chunks of layers and runs the interleaved one-forward-one-backward order;
    the weights after three steps, and after a checkpointed resume, are those of the single-process run."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={stages}", "--master-addr",
           "127.0.0.1", "--master-port", str(29676 + stages + 3 * virtual), os.path.join(ROOT, "tests", "mp", "mp_pipeline.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_PP_TIED=str(tied), SB_PP_MICRO=str(micro),
                                SB_PP_VIRTUAL=str(virtual), SB_PP_CKPT=str(tmp_path / "pp")))
    assert r.returncode == 0 and f"PIPELINE_OK stages={stages} virtual={virtual}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_interleaved_schedule_is_deadlock_free_in_order_and_shrinks_the_bubble():
    from scirust_b200.parallel.pipeline import check_schedule, interleaved_schedule
    for stages in (2, 3, 4, 8):
        for virtual in (1, 2, 3):
            for micro in (stages, 2 * stages, 4 * stages):
                check_schedule(stages, virtual, micro)                        # raises on deadlock / out-of-order delivery
                for rank in range(stages):
                    plan = interleaved_schedule(stages, virtual, micro, rank)
                    assert len(plan) == 2 * virtual * micro and len(set(plan)) == len(plan)
                    for kind in "FB":
                        for v in range(virtual):                             # per chunk: micro-batches in increasing order
                            ms = [m for k, c, m in plan if k == kind and c == v]
                            assert ms == sorted(ms) == list(range(micro))
                    done = set()
                    for k, c, m in plan:                                      # a backward never precedes its forward
                        assert k == "F" or ("F", c, m) in done
                        done.add((k, c, m))
    # one round = one chunk of work; a chunk is 1 / virtual of a stage, so compare rounds / virtual
    assert check_schedule(4, 2, 8) / 2 < check_schedule(4, 1, 8) and check_schedule(8, 3, 16) / 3 < check_schedule(8, 1, 16)
    with pytest.raises(ValueError):
        interleaved_schedule(4, 2, 6, 0)


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_equals_dense_attention_on_gloo_ranks(world):
    """Context parallelism: K/V shards travel around the ring, blocks are merged by log-sum-exp; forward output and
    the qkv gradient of every rank's slice equal dense attention over the whole sequence (causal and full)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29690 + world), os.path.join(ROOT, "tests", "mp", "mp_ring_attention.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode == 0 and "RING_ATTENTION_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_native_tcp_tree_allreduce_is_bitwise_the_python_engine_and_interoperates():
    """The C++ transport (csrc/rt_collectives.cpp) speaks the same frames and sums in the same order:
    all-native worlds, and worlds mixing native and Python ranks, give the in-process engine's bits."""
    for world, native_ranks in ((7, set(range(7))), (6, {0, 2, 5}), (2, {1})):
        xs = _inputs(world, 1000, seed=11)
        addrs = [("127.0.0.1", p) for p in _free_ports(world)]
        out, errs = [None] * world, []

        def work(r):
            try:
                fn = HC.tcp_tree_all_reduce_native if r in native_ranks else HC.tcp_tree_all_reduce_rank
                out[r] = fn(r, world, addrs, xs[r], timeout=20)
            except Exception as e:  # noqa: BLE001
                errs.append(e)
        ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert not errs, errs
        ref = HC.tree_all_reduce(xs)[0]
        assert all(np.array_equal(o, ref) for o in out)


def test_native_tcp_failures_are_errors_not_hangs():
    addrs = [("127.0.0.1", p) for p in _free_ports(3)]
    with pytest.raises(HC.CollectiveError, match="timed out"):
        HC.tcp_tree_all_reduce_native(0, 3, addrs, np.ones(4, np.float32), timeout=0.4)      # children never join
    with pytest.raises(HC.CollectiveError, match="timed out"):
        HC.tcp_tree_all_reduce_native(1, 3, addrs, np.ones(4, np.float32), timeout=0.4)      # parent never listens
    # a frame from a rank that is not a child is a protocol error
    addrs = [("127.0.0.1", p) for p in _free_ports(2)]
    res = {}

    def root():
        try:
            HC.tcp_tree_all_reduce_native(0, 2, addrs, np.ones(4, np.float32), timeout=5)
        except HC.CollectiveError as e:
            res["err"] = str(e)
    t = threading.Thread(target=root)
    t.start()
    for _ in range(200):
        try:
            s = socket.create_connection(addrs[0], timeout=1)
            break
        except OSError:
            import time
            time.sleep(0.02)
    HC.send_frame(s, 7, np.ones(4, np.float32).tobytes())
    t.join()
    s.close()
    assert "protocol" in res.get("err", "")


def test_flat_data_parallel_unused_parameter_and_accumulation():
    """A parameter without a gradient in a step contributes zero (not last step's gradient); a second backward
    before step() adds to the first (world 1, CPU statements of the cast and optimizer kernels)."""
    import torch.nn as nn
    from scirust_b200.parallel.ddp import FlatDataParallel

    class TwoHeads(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.trunk = nn.Linear(8, 8)
            self.a = nn.Linear(8, 4)
            self.b = nn.Linear(8, 4)

        def forward(self, x, use_b):
            h = torch.tanh(self.trunk(x))
            return (self.b(h) if use_b else self.a(h)).pow(2).mean()

    def run(dp_mode):
        m = TwoHeads()
        x = torch.randn(5, 8, generator=torch.Generator().manual_seed(1))
        if dp_mode:
            dp = FlatDataParallel(m, optimizer="sgd", lr=0.1, momentum=0.0)
        else:
            opt = torch.optim.SGD(m.parameters(), lr=0.1)
        for step in range(4):
            if dp_mode:
                dp(x, use_b=bool(step % 2)).backward()
                dp.step()
            else:
                opt.zero_grad(set_to_none=True)
                m(x, use_b=bool(step % 2)).backward()
                for p in m.parameters():          # bf16-rounded gradient, as the flat bf16 buffer holds it
                    if p.grad is not None:
                        p.grad = p.grad.to(torch.bfloat16).float()
                opt.step()
        return [p.detach().clone() for p in m.parameters()]

    for got, want in zip(run(True), run(False)):
        assert torch.allclose(got, want, atol=1e-6), (got - want).abs().max()

    # accumulation: two backward passes before step() == one backward of the summed loss (up to bf16 rounding)
    m = TwoHeads()
    dp = FlatDataParallel(m, optimizer="sgd", lr=0.1, momentum=0.0)
    x1 = torch.randn(5, 8, generator=torch.Generator().manual_seed(2))
    x2 = torch.randn(5, 8, generator=torch.Generator().manual_seed(3))
    with dp.no_sync():
        dp(x1, use_b=False).backward()
    dp(x2, use_b=False).backward()
    g_acc = dp.grad16.float().clone()
    dp.step()
    m2 = TwoHeads()
    (m2(x1, use_b=False) + m2(x2, use_b=False)).backward()
    ref = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in m2.parameters()])
    got = torch.cat([g_acc[o:o + p.numel()] for o, p in zip(dp.offs, dp.params)])
    assert torch.allclose(got, ref, atol=2e-2 * ref.abs().max().item() + 1e-6)
    assert got.abs().max() > 0


def test_fused_allreduce_refuses_more_buckets_than_it_has_counters():
    """The 257th bucket raises on the host; nothing is launched with an out-of-range counter pointer."""
    from scirust_b200.parallel import fused_allreduce as far

    class FakeRegion:
        rank, world = 0, 2
        slots = 0

        def flag_ptrs(self):
            return None

        def new_slot(self):
            FakeRegion.slots += 1
            return FakeRegion.slots - 1

        def peer_ptrs(self, t):
            return None

    src = torch.zeros(8 * 400, dtype=torch.bfloat16)
    ar = far.FusedAllReduce(FakeRegion(), src, src.clone())
    for i in range(far.FLAG_SLOTS):
        ar.bucket(8 * i, 8)
    with pytest.raises(RuntimeError, match="buckets"):
        ar.bucket(8 * far.FLAG_SLOTS, 8)


def test_multihost_proof_program_and_reduction_overhead_bench():
    """One process per rank over real TCP on the loopback; rank 0 recomputes the reference and must print PASS,
    for the fp32 fixed-order sum (Python and native transports) and the exact accumulator."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    for k, (combine, native) in enumerate((("fixed", 0), ("exact", 0), ("fixed", 1))):
        port0, port1 = 29490 + 4 * k, 29491 + 4 * k
        base = [sys.executable, "-m", "scirust_b200.parallel.proof_tcp_multihost", "--n", "4", "--dim", "3001",
                "--seed", "7", "--combine", combine, "--native", str(native)]
        procs = [subprocess.Popen(base + ["--rank", "0", "--my-addr", f"127.0.0.1:{port0}"], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True),
                 subprocess.Popen(base + ["--rank", "1", "--my-addr", f"127.0.0.1:{port1}", "--parent-addr",
                                          f"127.0.0.1:{port0}"], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.PIPE, text=True),
                 subprocess.Popen(base + ["--rank", "2", "--parent-addr", f"127.0.0.1:{port0}"], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True),
                 subprocess.Popen(base + ["--rank", "3", "--parent-addr", f"127.0.0.1:{port1}"], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)]
        outs = [p.communicate(timeout=120) for p in procs]
        assert all(p.returncode == 0 for p in procs), outs
        assert "verdict=PASS" in outs[0][0], outs[0]
        fps = {o[0].split("fingerprint=")[1].split()[0] for o in outs}
        assert len(fps) == 1
    # a root without a listener address is a usage error, not a hang
    r = subprocess.run([sys.executable, "-m", "scirust_b200.parallel.proof_tcp_multihost", "--rank", "0", "--n", "2"],
                       env=env, capture_output=True, text=True, timeout=60)
    assert r.returncode == 2
    from scirust_b200.parallel.bench_reduction_overhead import bench
    rows = bench(4096, [1, 3], 5)
    assert all(row["pinned_distinct_results"] == 1 for row in rows)


def test_rank_leaves_job_restarts_from_checkpoint_and_matches_uninterrupted_run(tmp_path):
    """Recovery: rank 1 leaves between steps, rank 0 gets PeerLost from the heartbeat, the supervisor restarts the job
    from the latest checkpoint, and the final loss and weights equal the uninterrupted run's bit for bit."""
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp"))
    from elastic_worker import worker
    from scirust_b200.train.elastic import EXIT_PEER_LOST, run_elastic

    a, b = tmp_path / "interrupted", tmp_path / "straight"
    a.mkdir()
    b.mkdir()
    hist = run_elastic(worker, 2, args=(str(a), 29540, 6, 1, 3), max_restarts=2, grace_s=30.0)
    assert len(hist) == 2 and hist[0][1] == 17 and hist[0][0] == EXIT_PEER_LOST and hist[1] == [0, 0]
    hist2 = run_elastic(worker, 2, args=(str(b), 29550, 6, -1, -1), max_restarts=0)
    assert hist2 == [[0, 0]]
    for r in range(2):
        assert (a / f"final_rank{r}.txt").read_text() == (b / f"final_rank{r}.txt").read_text()


def test_status_watchdog_reports_timeout_and_hang_without_a_gpu():
    import time
    from scirust_b200.ops._lib import CollectiveTimeout
    from scirust_b200.train.elastic import StatusWatchdog, StepHung
    code = {"v": 0}
    told = []
    wd = StatusWatchdog(lambda: code["v"], lambda: True, interval_s=0.02, hang_s=5.0, on_error=told.append).start()
    time.sleep(0.1)
    wd.check()
    code["v"] = 5                                  # a kernel recorded "peer flag never arrived"
    time.sleep(0.2)
    with pytest.raises(CollectiveTimeout):
        wd.check()
    assert len(told) == 1 and told[0].code == 5
    wd.stop()
    wd2 = StatusWatchdog(lambda: 0, lambda: False, interval_s=0.02, hang_s=0.1).start()
    wd2.arm()
    time.sleep(0.4)
    with pytest.raises(StepHung):
        wd2.check()
    wd2.stop()


@pytest.mark.parametrize("world,kv,vp", [(2, 2, 0), (2, 2, 1), (4, 2, 1)])
def test_tensor_parallel_training_on_the_host_backend_follows_the_single_device_model(world, kv, vp):
    """The tensor-parallel decoder (and its vocabulary-parallel variant: sharded embedding, LM head and cross-entropy)
    on gloo ranks with CPU tensors: losses and trained shards follow the single-device model, replicated parameters
    stay identical on every rank. With 4 ranks and 2 KV heads each KV head is replicated over a group of 2 ranks."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + 3 * world + vp), os.path.join(ROOT, "tests", "mp", "mp_tp_model_host.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_TP_KV=str(kv), SB_TP_VOCAB_PARALLEL=str(vp)))
    assert r.returncode == 0 and f"TP_HOST_OK world={world} kv={kv} vp={vp}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("dp,tp,vp", [(2, 2, 0), (2, 4, 1)])
def test_data_parallel_times_tensor_parallel_on_a_mesh_of_gloo_ranks(dp, tp, vp):
    """A ("dp", "tp") mesh: tensor-parallel groups are runs of consecutive ranks, replicas differ in their batch, the
    gradient is summed over the data-parallel axis. With tp = 4 and 2 KV heads the replicated KV projections are reduced
    inside sub-groups of each tensor-parallel group. Result: the single-device model trained on the whole batch."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={dp * tp}", "--master-addr",
           "127.0.0.1", "--master-port", str(29720 + dp * tp + vp), os.path.join(ROOT, "tests", "mp", "mp_dp_tp_host.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1200,
                       env=dict(os.environ, PYTHONPATH=ROOT, SB_DP=str(dp), SB_TP=str(tp), SB_TP_VOCAB_PARALLEL=str(vp)))
    assert r.returncode == 0 and f"DP_TP_HOST_OK dp={dp} tp={tp} vp={vp}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
