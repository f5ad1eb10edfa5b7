"""Decode-time kernels and the inference engine against fp32 PyTorch references."""
import pytest
import torch

from scirust_b200.models import GQADecoder, SciAgentConfig
from scirust_b200.models.infer import InferenceEngine, reference_generate
from scirust_b200.ops import _lib, decode as D

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _r(shape, seed, scale=0.5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(BF)


@pytest.mark.parametrize("M,K,N", [(1, 1024, 1536), (3, 4096, 512), (8, 2816, 1024), (13, 1024, 264),
                                   (8, 14336, 520), (2, 40, 8), (1, 4096, 6144), (16, 4096, 1024), (27, 2816, 520),
                                   (32, 14336, 256), (45, 1024, 512)])
def test_gemv_bf16(M, K, N):
    x, w, r = _r((M, K), 1), _r((K, N), 2), _r((M, N), 3)
    y = D.gemv(x, w, residual=r)
    ref = x.float() @ w.float() + r.float()
    assert (y.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert torch.equal(y, D.gemv(x, w, residual=r))
    f = torch.empty((M, N), dtype=torch.float32, device="cuda")
    D.gemv(x, w, out_f32=f)
    assert (f - x.float() @ w.float()).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,K,N", [(1, 1024, 1536), (5, 4096, 512), (8, 1024, 2048), (7, 14336, 528)])
def test_gemv_int8_and_quantize(M, K, N):
    x, w = _r((M, K), 4), _r((K, N), 5)
    qw = D.quantize_per_channel(w)
    qc = D.quantize_per_channel(w.cpu())
    assert torch.allclose(qw.scale.cpu(), qc.scale, rtol=1e-6)
    assert (qw.q.cpu().int() - qc.q.int()).abs().max().item() <= 1   # bf16 half-way cases may round either way
    y = D.gemv(x, qw)
    ref = x.float() @ (qw.q.float() * qw.scale[None, :])
    assert (y.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert (qw.dequantize().float() - qw.q.float() * qw.scale[None, :]).abs().max().item() <= 1e-2


@pytest.mark.parametrize("dh,H,Hkv", [(64, 16, 4), (128, 32, 8), (128, 4, 4), (64, 16, 2), (128, 16, 1)])
def test_paged_decode_attention(dh, H, Hkv):
    B, page, max_seq = 3, 16, 700
    max_blocks = (max_seq + page - 1) // page
    n_blocks = B * max_blocks
    pool = torch.zeros((n_blocks, 2, Hkv, page, dh), dtype=BF, device="cuda")
    perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(0)).int()
    table = perm.reshape(B, max_blocks).cuda()          # scattered physical pages
    lens = torch.tensor([1, 257, 700], dtype=torch.int32, device="cuda")
    ld = (H + 2 * Hkv) * dh
    for b in range(B):
        L = int(lens[b])
        rows = _r((L, ld), 10 + b)
        D.kv_append(rows, H, Hkv, dh, pool, table, page, torch.full((L,), b, dtype=torch.int32, device="cuda"),
                    torch.arange(L, dtype=torch.int32, device="cuda"))
    q = _r((B, ld), 20)
    out = D.decode_attention(q, pool, table, page, lens, H, Hkv, dh, n_splits=5)
    ref = D.decode_attention_ref(q, pool, table, page, lens, H, Hkv, dh)
    assert (out.float() - ref).abs().max().item() < 2e-2
    one = D.decode_attention(q, pool, table, page, lens, H, Hkv, dh, n_splits=1)
    assert (one.float() - ref).abs().max().item() < 2e-2
    assert torch.equal(out, D.decode_attention(q, pool, table, page, lens, H, Hkv, dh, n_splits=5))


def test_argmax_tie_and_nan_rules():
    V = 10000
    lg = torch.randn(8, V, device="cuda")
    lg[0, 77] = 50.0
    lg[0, 9000] = 50.0          # tie -> lower id
    lg[1, 5] = float("nan")     # a NaN past column 0 is skipped
    lg[1, 4100] = 60.0
    lg[2] = -5.0
    lg[2, 8191] = -4.0
    lg[4, 0] = float("nan")     # NaN in column 0: the greedy loop starts from it and nothing compares greater
    lg[4, 300] = 99.0
    lg[5, 4096] = float("nan")  # first element of the second slab
    lg[5, 4097] = 70.0
    lg[6] = float("nan")        # no number at all
    lg[7, 4096] = float("nan")  # the maximum sits in the first slab, the second slab starts with a NaN
    lg[7, 17] = 80.0
    tok = D.argmax_rows(lg).tolist()
    assert tok[:3] == [77, 4100, 8191]
    assert tok[3] == int(torch.argmax(lg[3]))
    assert tok[4:] == [0, 4097, 0, 17]
    # the host statement of the same rule agrees row by row
    assert D.argmax_rows(lg.cpu()).tolist() == tok


@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("M,K,N,splits", [(1, 1024, 50272, 1), (5, 2048, 4112, 4), (8, 512, 1024, None)])
def test_lm_head_fused_with_argmax_equals_gemv_then_argmax(quant, M, K, N, splits):
    """One launch (GEMV + in-kernel arg-max) gives the tokens and the logits of the three-launch path, including the
    NaN rules: weights with NaN columns make NaN logits in column 0 (row wins token 0), column 7 (skipped)."""
    g = torch.Generator(device="cuda").manual_seed(M * 31 + K)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(K, N, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    gain = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).to(torch.bfloat16)
    w[:, N - 3] = w[:, 40]                          # a tie between two columns when x.w is the row maximum
    cases = [w]
    if not quant:
        wn = w.clone(); wn[0, 7] = float("nan"); cases.append(wn)           # NaN logits in column 7: skipped
        w0 = w.clone(); w0[0, 0] = float("nan"); cases.append(w0)           # NaN logits in column 0: token 0
    for wc in cases:
        wt = D.quantize_per_channel(wc) if quant else wc
        lg = torch.empty(M, N, dtype=torch.float32, device="cuda")
        D.gemv(x, wt, out_f32=lg, rms_weight=gain, splits=splits)
        want = D.argmax_rows(lg)
        lg2 = torch.zeros_like(lg)
        got = D.gemv_argmax(x, wt, rms_weight=gain, logits=lg2, splits=splits)
        nolog = D.gemv_argmax(x, wt, rms_weight=gain, splits=splits)
        torch.cuda.synchronize()
        assert torch.equal(got, want) and torch.equal(nolog, want)
        nan = torch.isnan(lg)
        assert torch.equal(torch.isnan(lg2), nan) and torch.equal(lg2[~nan], lg[~nan])
    if not quant:
        assert got.tolist() == [0] * M
    from scirust_b200.ops import _lib
    _lib.check_status(torch.device("cuda"))


@pytest.mark.parametrize("quant", [None, "int8"])
def test_engine_cached_equals_naive_and_graph(quant):
    cfg = SciAgentConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, d_ff=512,
                         max_seq_len=512, rope_theta=10000.0)
    model = GQADecoder(cfg, device="cuda", seed=5, init_std=0.08)
    prompts = torch.randint(1, 1024, (2, 128), generator=torch.Generator().manual_seed(1)).cuda()
    eager = InferenceEngine(model, quant=quant, max_batch=2, max_seq=256, page=16, use_graph=False)
    graph = InferenceEngine(model, quant=quant, max_batch=2, max_seq=256, page=16, use_graph=True)
    a = eager.generate(prompts, 8)
    b = graph.generate(prompts, 8)
    _lib.check_status()
    assert torch.equal(a, b)
    if quant is None:
        naive = reference_generate(model, prompts, 8)
        assert torch.equal(a, naive), (a.tolist(), naive.tolist())


@pytest.mark.parametrize("M,K,N", [(16, 1024, 512), (64, 4096, 1536), (200, 1000, 272), (2048, 1024, 2816)])
def test_dequant_fused_gemm(M, K, N):
    x, w, r = _r((M, K), 6), _r((K, N), 7), _r((M, N), 8)
    qw = D.quantize_per_channel(w)
    ref = x.float() @ (qw.q.float() * qw.scale[None, :]) + r.float()
    y = D.matmul_w8(x, qw, residual=r)
    _lib.check_status()
    assert (y.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    y2 = D.matmul_w8(x, qw, residual=r, splits=4)
    _lib.check_status()
    assert (y2.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    assert torch.equal(y2, D.matmul_w8(x, qw, residual=r, splits=4))


@pytest.mark.parametrize("M,K,N,splits", [(16, 4096, 1024, None), (64, 512, 768, 1), (200, 1040, 264, 3), (9, 128, 8, None)])
def test_w8a8_gemm_on_integer_tensor_cores_is_exact(M, K, N, splits):
    """tcgen05.mma.kind::i8: int8 x int8 -> int32 is exact, so the kernel must reproduce the host statement of the
    reference's quantised linear layer (dynamic row scales, int64 accumulation, one rescale) to the last bf16 bit,
    whatever the split-K factor; and it stays close to the unquantised product."""
    g = torch.Generator(device="cuda").manual_seed(M + K)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.7).to(torch.bfloat16)
    w = (torch.randn(K, N, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    r = (torch.randn(M, N, generator=g, device="cuda") * 0.3).to(torch.bfloat16)
    wq = D.quantize_per_channel(w)
    xq, sx = D.quantize_rows(x)
    xq_ref, sx_ref = D.quantize_rows(x.cpu())
    assert torch.equal(xq.cpu(), xq_ref) and torch.equal(sx.cpu(), sx_ref)
    acc = xq.cpu().to(torch.int64) @ wq.q.cpu().to(torch.int64)
    want = (acc.float() * (sx_ref[:, None] * wq.scale.cpu()[None, :]) + r.cpu().float()).to(torch.bfloat16)
    got = D.matmul_w8a8(x, wq, residual=r, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), want)
    again = D.matmul_w8a8(x, wq, residual=r, splits=2 if K >= 256 else 1)
    assert torch.equal(again, got)                        # split-K adds integers: same bits
    full = x.float() @ w.float() + r.float()
    assert (got.float() - full).abs().max().item() <= 0.04 * full.abs().max().item()
    from scirust_b200.ops import _lib
    _lib.check_status(torch.device("cuda"))


@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("M,K,N,splits", [(16, 4096, 1024, 0), (9, 320, 264, 1), (33, 1040, 4104, 3), (64, 512, 128, 0),
                                          (12, 128, 19200, 0)])
def test_skinny_weight_streaming_gemm_matches_reference(quant, M, K, N, splits):
    """9..64 rows on the swapped-operand tcgen05 kernel (weights as the 128-row operand, C^T in tensor memory):
    bf16 against the fp32 product, int8 (W8A8) bit for bit against the integer statement; ragged N and K, one and
    several work items per CTA, explicit and automatic split-K; two runs agree bit for bit."""
    if quant and K % 16:
        K = (K + 15) // 16 * 16
    g = torch.Generator(device="cuda").manual_seed(M * 7 + K)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.7).to(torch.bfloat16)
    w = (torch.randn(K, N, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    r = (torch.randn(M, N, generator=g, device="cuda") * 0.3).to(torch.bfloat16)
    if quant:
        wq = D.quantize_per_channel(w)
        xq, sx = D.quantize_rows(x.cpu())
        acc = xq.to(torch.int64) @ wq.q.cpu().to(torch.int64)
        want = (acc.float() * (sx[:, None] * wq.scale.cpu()[None, :]) + r.cpu().float()).to(torch.bfloat16)
        got = D.matmul_skinny(x, wq, residual=r, splits=splits)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want)
        assert torch.equal(D.matmul_skinny(x, wq, residual=r, splits=splits), got)
    else:
        ref = x.float() @ w.float() + r.float()
        got = D.matmul_skinny(x, w, residual=r, splits=splits)
        torch.cuda.synchronize()
        err = (got.float() - ref).abs()
        tol = ref.abs() * 2.0 ** -7 + 2.0 ** -14 * 0.035 * 0.8 * K + 1e-3
        assert bool((err <= tol).all()), float((err - tol).max())
        assert torch.equal(D.matmul_skinny(x, w, residual=r, splits=splits), got)
        plain = D.matmul_skinny(x, w, splits=1)
        assert (plain.float() - x.float() @ w.float()).abs().max().item() <= 0.02 * max(1.0, (x.float() @ w.float()).abs().max().item())
    from scirust_b200.ops import _lib
    _lib.check_status(torch.device("cuda"))


def test_driver_smoke_entry_runs_training_decode_and_batched_decode():
    """The entry point the round-end driver calls: a few training steps, a cached decode, and 12-sequence decodes with
    bf16 and int8 weights (the weight-streaming GEMM and its W8A8 form)."""
    import __graft_entry__ as entry
    entry.smoke()
