"""Numerics of every CUDA kernel against the PyTorch fp32 restatement of the same op.

Sweeps follow the reference's kernel tests (gemv/src/test_batch_decode.cu:190-217 batch / head /
head_dim / sm_blk sweeps; gemv/src/test_batch_prefill.cu:467-554 short and long contexts;
cutlassGemmWrapperImpl.cuh:333-372 GEMM self-check) with tighter tolerances.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from nanoflow_b200 import ops
from nanoflow_b200.ops import reference as ref


def _close(got, want, atol, rtol, frac=1.0):
    got, want = got.float(), want.float()
    assert not torch.isnan(got).any(), "NaN in kernel output"
    ok = (got - want).abs() <= atol + rtol * want.abs()
    assert int(ok.sum().item()) >= frac * ok.numel(), (
        f"{(~ok).sum().item()} / {ok.numel()} mismatches, max err {(got - want).abs().max().item()}")


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (77, 264, 200),
                                   (1, 128, 128), (640, 1280, 8192), (1408, 1024, 1024),
                                   (300, 8192, 3584)])
@pytest.mark.parametrize("tile_n", [0, 32, 64, 96, 128, 160, 192, 224, 256])
def test_gemm_plain(M, N, K, tile_n):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    st = ops.new_status()
    out = ops.gemm(a, w, tile_n=tile_n, status=st)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w), atol=2e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(256, 8192, 8192), (85, 1024, 3584), (300, 2048, 4096), (512, 4096, 1024),
                                   (129, 10240, 2048)])
@pytest.mark.parametrize("tile_m,tile_n,split_k", [(0, 0, 0), (2, 256, 1), (2, 256, 4), (4, 128, 3), (1, 256, 2),
                                                   (4, 64, 1), (2, 128, 8), (1, 128, 5), (1, 64, 2), (2, 224, 3),
                                                   (2, 160, 1), (4, 96, 2)])
def test_gemm_small_m_weight_streaming(M, N, K, tile_m, tile_n, split_k):
    """Multi-M-tile CTAs (weights fetched once) and split-K with fp32 partials + reduce pass."""
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(64 << 20, device="cuda", dtype=torch.float32)
    st = ops.new_status()
    want = ref.gemm(a, w, res, 0.5, bias)
    out = ops.gemm(a, w, residual=res, beta=0.5, bias=bias, tile_m=tile_m, tile_n=tile_n,
                   split_k=split_k, workspace=ws, status=st)
    ops.check_status(st, "gemm")
    _close(out, want, atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(2048, 1280, 2048), (640, 1280, 1024), (1408, 8192, 512), (1000, 3000, 1000)])
@pytest.mark.parametrize("num_ctas", [0, 100, 37])
def test_gemm_split_k_large(M, N, K, num_ctas):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(64 << 20, device="cuda", dtype=torch.float32)
    st = ops.new_status()
    out = ops.gemm(a, w, residual=res, beta=1.0, split_k=3, workspace=ws, num_ctas=num_ctas, status=st)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 1.0), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)
    out0 = ops.gemm(a, w, residual=res, beta=1.0, workspace=ws, num_ctas=num_ctas)   # chooser
    _close(out0, ref.gemm(a, w, res, 1.0), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,F,K,tile_m,tile_n", [(256, 3584, 1024, 2, 256), (200, 1792, 2048, 2, 128),
                                                 (500, 1024, 1024, 4, 128), (256, 28672 // 8, 8192, 0, 0),
                                                 (256, 3584, 1024, 2, 224), (300, 1000, 512, 2, 192)])
def test_gemm_swiglu_small_m(M, F, K, tile_m, tile_n):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ws = torch.zeros(80 << 20, device="cuda", dtype=torch.float32)
    st = ops.new_status()
    want = ref.gemm_swiglu(a, wg, wu)
    out = ops.gemm_swiglu(a, wg, wu, tile_m=tile_m, tile_n=tile_n, status=st)
    ops.check_status(st, "gemm_swiglu")
    _close(out, want, atol=3e-2 * math.sqrt(K / 64), rtol=3e-2)



@pytest.mark.parametrize("num_ctas", [1, 7, 60, 148])
def test_gemm_cta_budget_residual_bias(num_ctas):
    M, N, K = 520, 1032, 328
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    st = ops.new_status()
    out = ops.gemm(a, w, residual=res, beta=0.125, bias=bias, num_ctas=num_ctas, status=st)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 0.125, bias), atol=5e-2, rtol=2e-2)


def test_gemm_strided_views_and_inplace_residual():
    M, N, K = 200, 512, 256
    big_a = torch.randn(M, 2 * K, device="cuda", dtype=torch.bfloat16)
    a = big_a[:, K:]
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    big_out = torch.randn(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    want = ref.gemm(a, w, big_out[:, :N], 1.0)
    ops.gemm(a, w, out=big_out[:, :N], residual=big_out[:, :N], beta=1.0)
    _close(big_out[:, :N], want, atol=5e-2, rtol=2e-2)


def test_gemm_reduced_smem_budget():
    """A smaller shared-memory budget (fewer TMA stages) leaves room for a co-resident kernel."""
    a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16) * 0.05
    want = ref.gemm(a, w)
    for kb in (0, 160, 128, 100):
        _close(ops.gemm(a, w, tile_n=256, smem_budget_kb=kb), want, atol=0.1, rtol=2e-2)
    with pytest.raises(RuntimeError):
        ops.gemm(a, w, tile_n=256, smem_budget_kb=60)          # not even two stages fit


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (384, 768, 512), (200, 264, 192), (1000, 1000, 1024),
                                   (2048, 1280, 1024), (130, 40, 64), (3712, 1280, 512)])
@pytest.mark.parametrize("tile_n,split_k,num_ctas", [(256, 1, 0), (128, 1, 0), (224, 2, 0), (64, 1, 37),
                                                     (32, 1, 0), (160, 3, 100), (256, 1, 2)])
def test_gemm_cta_pair(M, N, K, tile_n, split_k, num_ctas):
    """tcgen05.mma.cta_group::2: two CTAs of a cluster share a 256-row tile (odd tile counts, ragged
    edges, split-K, restricted CTA budgets)."""
    if split_k > 1 and K // 64 < split_k:
        pytest.skip("fewer k-blocks than splits")
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(64 << 20, device="cuda", dtype=torch.float32)
    st = ops.new_status()
    out = ops.gemm(a, w, residual=res, beta=0.5, bias=bias, tile_m=1, tile_n=tile_n, split_k=split_k,
                   workspace=ws, num_ctas=num_ctas, cta_group=2, status=st)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 0.5, bias), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(4096, 1280, 1024), (1000, 1000, 512), (3712, 8192, 256), (130, 40, 64)])
@pytest.mark.parametrize("tile_m,tile_n,cta_group,split_k", [(0, 0, 0, 0), (1, 256, 2, 1), (1, 128, 2, 2), (1, 128, 1, 1),
                                                             (2, 96, 1, 3)])
def test_gemm_work_units_dealt_by_the_block_scheduler(M, N, K, tile_m, tile_n, cta_group, split_k):
    """stream_k = 3: one work unit per CTA (or CTA pair) and more CTAs than fit on the GPU at once; the result is
    that of the persistent launch."""
    if split_k > 1 and K // 64 < split_k:
        pytest.skip("fewer k-blocks than splits")
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(max(64 << 20, max(split_k, 1) * M * N), device="cuda", dtype=torch.float32)
    st = ops.new_status()
    kw = dict(residual=res, beta=0.5, bias=bias, tile_m=tile_m, tile_n=tile_n, split_k=split_k, workspace=ws,
              cta_group=cta_group, status=st)
    out = ops.gemm(a, w, stream_k=3, **kw)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 0.5, bias), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)
    assert torch.equal(out, ops.gemm(a, w, stream_k=2, **kw))
    f = 1792
    wg = torch.randn(f, K, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(f, K, device="cuda", dtype=torch.bfloat16) * 0.05
    if split_k <= 1:
        act = ops.gemm_swiglu(a, wg, wu, tile_m=tile_m, tile_n=tile_n, cta_group=cta_group, stream_k=3, workspace=ws, status=st)
        ops.check_status(st, "gemm_swiglu")
        assert torch.equal(act, ops.gemm_swiglu(a, wg, wu, tile_m=tile_m, tile_n=tile_n, cta_group=cta_group, stream_k=2,
                                                workspace=ws, status=st))


@pytest.mark.parametrize("M,N,K", [(256, 320, 64), (4096, 1280, 512), (1000, 1000, 1024), (300, 2048, 192), (130, 40, 64),
                                   (3712, 1280, 256)])
@pytest.mark.parametrize("tile_n,split_k,num_ctas", [(320, 1, 0), (384, 1, 0), (448, 2, 0), (512, 1, 0), (320, 1, 6)])
def test_gemm_cta_pair_tiles_wider_than_one_mma(M, N, K, tile_n, split_k, num_ctas):
    """CTA pairs on 256 x tile_n tiles with tile_n > 256: two pair MMAs of tile_n / 2 columns per k step into one
    accumulator, each CTA staging a quarter of the tile's weight rows per MMA (ragged edges, a tile that is mostly
    past the last column, split-K, a restricted CTA budget)."""
    if split_k > 1 and K // 64 < split_k:
        pytest.skip("fewer k-blocks than splits")
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(max(64 << 20, split_k * M * N), device="cuda", dtype=torch.float32)
    st = ops.new_status()
    out = ops.gemm(a, w, residual=res, beta=0.5, bias=bias, tile_m=1, tile_n=tile_n, split_k=split_k,
                   workspace=ws, num_ctas=num_ctas, cta_group=2, status=st)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 0.5, bias), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)
    # the same product through the 256-wide pair tiles, bit for bit (same k order per output element)
    if split_k == 1:
        assert torch.equal(out, ops.gemm(a, w, residual=res, beta=0.5, bias=bias, tile_m=1, tile_n=256, split_k=1,
                                         workspace=ws, cta_group=2, stream_k=2, status=st))


def test_gemm_wide_tiles_need_a_cta_pair():
    a = torch.randn(256, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(640, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.gemm(a, w, tile_m=1, tile_n=320, cta_group=1)
    with pytest.raises(RuntimeError):
        ops.gemm_swiglu(a, w, w, tile_m=1, tile_n=320, cta_group=2)


@pytest.mark.parametrize("M,F,K", [(256, 128, 64), (300, 3584, 1024), (1408, 1792, 2048), (129, 264, 136)])
@pytest.mark.parametrize("tile_n", [128, 192, 224, 256])
def test_gemm_swiglu_cta_pair(M, F, K, tile_n):
    """CTA pair with the SwiGLU epilogue: one CTA stages the gate rows, its peer the up rows."""
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    st = ops.new_status()
    out = ops.gemm_swiglu(a, wg, wu, tile_m=1, tile_n=tile_n, cta_group=2, status=st)
    ops.check_status(st, "gemm_swiglu")
    _close(out, ref.gemm_swiglu(a, wg, wu), atol=3e-2 * math.sqrt(K / 64), rtol=3e-2)


@pytest.mark.parametrize("M,N,K,tile_m,tile_n,cta_group,num_ctas", [
    (256, 8192, 1024, 2, 256, 1, 0),      # 32 tiles on 148 workers: every tile is cut into k ranges
    (256, 8192, 1024, 1, 256, 2, 0),
    (256, 8192, 2048, 1, 128, 1, 0),
    (300, 4096, 1536, 4, 128, 1, 0),
    (2048, 1280, 2048, 1, 256, 2, 0),
    (3712, 1280, 1024, 1, 256, 2, 0),     # 75 pair tiles on 74 pairs: one left over, cut 16 ways
    (3712, 1280, 1024, 1, 256, 1, 0),
    (1000, 3000, 1024, 1, 224, 1, 37),
    (1000, 3000, 1024, 1, 160, 2, 36),
    (130, 1000, 4096, 2, 96, 1, 0),
])
def test_gemm_stream_k_tail(M, N, K, tile_m, tile_n, cta_group, num_ctas):
    """Left-over tiles of the last wave cut into k-block ranges (fp32 partial copies + second pass);
    twice through the same workspace."""
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    for _ in range(2):
        res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        st = ops.new_status()
        out = ops.gemm(a, w, residual=res, beta=0.5, bias=bias, tile_m=tile_m, tile_n=tile_n, workspace=ws,
                       cta_group=cta_group, num_ctas=num_ctas, stream_k=1, status=st)
        ops.check_status(st, "gemm")
        _close(out, ref.gemm(a, w, res, 0.5, bias), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)


@pytest.mark.parametrize("M,F,K,tile_m,tile_n,cta_group", [(256, 3584, 1024, 2, 256, 1), (256, 3584, 2048, 1, 224, 2),
                                                            (1408, 1792, 1024, 1, 256, 2), (300, 7168, 512, 1, 192, 1)])
def test_gemm_swiglu_stream_k_tail(M, F, K, tile_m, tile_n, cta_group):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ws = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    st = ops.new_status()
    out = ops.gemm_swiglu(a, wg, wu, tile_m=tile_m, tile_n=tile_n, cta_group=cta_group, workspace=ws,
                          stream_k=1, status=st)
    ops.check_status(st, "gemm_swiglu")
    _close(out, ref.gemm_swiglu(a, wg, wu), atol=3e-2 * math.sqrt(K / 64), rtol=3e-2)


def test_gemm_cta_pair_rejects_multi_tile_ctas():
    a = torch.randn(256, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(128, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.gemm(a, w, tile_m=2, tile_n=128, cta_group=2)


@pytest.mark.parametrize("M,N,K,kw", [
    (256, 8192, 1024, dict(split_k=4, tile_m=2, tile_n=256)),       # norm out of the split-K reduce pass
    (100, 1024, 2048, dict(split_k=3, tile_m=1, tile_n=128)),
    (256, 4096, 8192, dict()),                                       # the cost model's shape
    (1000, 1024, 512, dict(split_k=1, tile_m=1, tile_n=256)),       # not split: norm launch after the GEMM
    (512, 2048, 1024, dict(cta_group=2, tile_m=1, tile_n=256, stream_k=1)),
])
def test_gemm_with_rmsnorm_of_result(M, N, K, kw):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    nw = 1.0 + 0.1 * torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(64 << 20, device="cuda", dtype=torch.float32)
    normed = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    st = ops.new_status()
    out = ops.gemm(a, w, residual=res, beta=1.0, workspace=ws, status=st, norm_w=nw, norm_out=normed, norm_eps=1e-5,
                   **kw)
    ops.check_status(st, "gemm")
    _close(out, ref.gemm(a, w, res, 1.0), atol=3e-2 * math.sqrt(K / 64), rtol=2e-2)
    # the norm is taken on the stored (bf16) rows, as a separate norm kernel would
    _close(normed, ref.rmsnorm(out, nw, 1e-5), atol=2e-2, rtol=2e-2)


def test_gemm_empty_and_bad_args():
    a = torch.randn(0, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(128, 64, device="cuda", dtype=torch.bfloat16)
    assert ops.gemm(a, w).shape == (0, 128)
    with pytest.raises(RuntimeError):
        ops.gemm(torch.randn(8, 60, device="cuda", dtype=torch.bfloat16),
                 torch.randn(128, 60, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (300, 3584, 1024), (1408, 1792, 4096), (17, 264, 136)])
@pytest.mark.parametrize("tile_n", [0, 128, 192, 224, 256])
def test_gemm_swiglu(M, F, K, tile_n):
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.05
    st = ops.new_status()
    out = ops.gemm_swiglu(a, wg, wu, tile_n=tile_n, status=st)
    ops.check_status(st, "gemm_swiglu")
    _close(out, ref.gemm_swiglu(a, wg, wu), atol=3e-2 * math.sqrt(K / 64), rtol=3e-2)


@pytest.mark.parametrize("rows,cols", [(1, 256), (37, 4096), (640, 8192), (5, 1032)])
def test_rmsnorm(rows, cols):
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(cols, device="cuda", dtype=torch.bfloat16)
    _close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x, w, 1e-5), atol=2e-2, rtol=2e-2)
    resid = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    r0 = resid.clone()
    out = ops.add_rmsnorm(resid, x, w, 1e-5)
    newres = (r0.float() + x.float()).bfloat16()
    _close(resid, newres, atol=1e-2, rtol=1e-2)
    _close(out, ref.rmsnorm(newres, w, 1e-5), atol=2e-2, rtol=2e-2)


def test_embedding_feedback_and_gather():
    vocab, hidden, n = 1000, 512, 50
    table = torch.randn(vocab, hidden, device="cuda", dtype=torch.bfloat16)
    host_ids = torch.randint(0, vocab, (n,), device="cuda", dtype=torch.int32)
    prev = torch.randint(0, vocab, (20,), device="cuda", dtype=torch.int32)
    src = torch.full((n,), -1, device="cuda", dtype=torch.int32)
    src[:15] = torch.randperm(20, device="cuda")[:15].int()
    ids_out = torch.empty(n, device="cuda", dtype=torch.int32)
    st = ops.new_status()
    out = ops.embedding(table, host_ids, feedback_src=src, prev_tokens=prev, ids_out=ids_out, status=st)
    want_ids = torch.where(src >= 0, prev[src.clamp(min=0).long()], host_ids)
    assert torch.equal(ids_out, want_ids)
    assert torch.equal(out, table[want_ids.long()])
    ops.check_status(st)
    # out-of-range id is clamped and reported, never dereferenced
    bad = host_ids.clone(); bad[3] = vocab + 5
    ops.embedding(table, bad, status=st)
    with pytest.raises(RuntimeError):
        ops.check_status(st)
    idx = torch.tensor([4, 0, 49, 7], device="cuda", dtype=torch.int32)
    assert torch.equal(ops.gather_rows(out, idx), out[idx.long()])


def test_small_elementwise():
    g = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
    u = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
    _close(ops.silu_mul(g, u), ref.silu_mul(g, u), atol=2e-2, rtol=2e-2)
    assert torch.equal(ops.transpose(g), g.t().contiguous())
    dst = torch.zeros(64, 256, device="cuda", dtype=torch.bfloat16)
    ops.copy_cols(dst, g[:, 512:768])
    assert torch.equal(dst, g[:, 512:768])


@pytest.mark.parametrize("rows,cols", [(1, 32000), (37, 128256), (300, 1000), (8, 152064 // 8)])
def test_argmax(rows, cols):
    logits = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    val = torch.empty(rows, device="cuda", dtype=torch.float32)
    idx = ops.argmax(logits, col_offset=100, val_out=val)
    # bf16 ties: the kernel returns the lowest index of the maximum
    mx = logits.float().max(dim=-1).values
    first = (logits.float() == mx[:, None]).int().argmax(dim=-1).int()
    assert torch.equal(idx, first + 100)
    assert torch.equal(val, mx)
    # sharded combine
    shards = 4
    per = cols // shards // 8 * 8
    cv = torch.empty(shards, rows, device="cuda", dtype=torch.float32)
    ci = torch.empty(shards, rows, device="cuda", dtype=torch.int32)
    for s in range(shards):
        ops.argmax(logits[:, s * per:(s + 1) * per], col_offset=s * per, idx_out=ci[s], val_out=cv[s])
    full = ops.argmax(logits[:, :shards * per])
    assert torch.equal(ops.argmax_combine(cv, ci), full)


def test_flags_and_sleep():
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    st = ops.new_status()
    ops.flag_add(flag, 3)
    ops.flag_wait(flag, 3, 1000, st)
    ops.check_status(st)
    ops.flag_clear(flag)
    # a wait nobody satisfies runs out after its limit and reports, leaving the context usable
    ops.flag_wait(flag, 1, 2000, st)
    with pytest.raises(RuntimeError):
        ops.check_status(st)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); ops.sleep_us(2000); e1.record(); torch.cuda.synchronize()
    assert 1.5 <= e0.elapsed_time(e1) <= 50


def _make_paged(batch_lens, qo_lens, kv_heads, hd, page=16, extra_pages=5, shuffle=True):
    """Random paged pool + metadata for requests with given kv lengths (after append)."""
    npages = [(l + page - 1) // page for l in batch_lens]
    total = sum(npages) + extra_pages
    perm = torch.randperm(total) if shuffle else torch.arange(total)
    kv_indptr = [0]
    for n in npages:
        kv_indptr.append(kv_indptr[-1] + n)
    kv_indices = perm[:kv_indptr[-1]].int()
    last = [(l - 1) % page + 1 for l in batch_lens]
    qo_indptr = [0]
    for n in qo_lens:
        qo_indptr.append(qo_indptr[-1] + n)
    pool = torch.randn(total, 2, kv_heads, page, hd, device="cuda", dtype=torch.bfloat16)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return pool, dev(qo_indptr), dev(kv_indptr), kv_indices.cuda(), dev(last)


@pytest.mark.parametrize("batch", [1, 7, 37, 61, 300])
@pytest.mark.parametrize("kv_heads,group", [(8, 8), (1, 8), (4, 4), (2, 1), (1, 16)])
@pytest.mark.parametrize("num_ctas,stages", [(0, 0), (7, 2), (30, 4), (3, 3)])
def test_attn_decode_tma_producer(batch, kv_heads, group, num_ctas, stages):
    """The decode kernel with a TMA producer warp (one work item per consumer warp, pages through an mbarrier
    ring): same results as the fp32 restatement for every ring depth and CTA budget."""
    hd = 128
    q_heads = kv_heads * group
    lens = torch.randint(1, 700, (batch,)).tolist()
    lens[0] = 1
    if batch > 2:
        lens[1], lens[2] = 16, 17
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    st = ops.new_status()
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                    num_ctas=num_ctas, status=st, stages=stages, impl="tma")
    ops.check_status(st, "attn_decode tma")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)


def test_attn_decode_tma_forwards_split_kv_and_request_ranges():
    """chunk_pages > 0 goes to the kernel with the merge pass; req_begin selects a range of requests."""
    kv_heads, group, hd, batch = 2, 8, 128, 9
    q_heads = kv_heads * group
    lens = [2000, 31, 4096, 640, 1, 99, 100, 515, 16]
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    out = torch.zeros_like(q)
    ws = torch.empty(batch * q_heads * 16 * (hd + 2), device="cuda", dtype=torch.float32)
    st = ops.new_status()
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                    chunk_pages=16, workspace=ws, max_chunks=16, status=st, impl="tma")
    ops.check_status(st, "attn_decode tma split")
    _close(out, want, atol=1e-2, rtol=2e-2)
    out2 = torch.zeros_like(q)
    ops.attn_decode(q, out2, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=3, req_count=4, status=st, impl="tma")
    ops.check_status(st, "attn_decode tma range")
    _close(out2[3:7], want[3:7], atol=1e-2, rtol=2e-2)
    assert bool((out2[:3] == 0).all()) and bool((out2[7:] == 0).all())


@pytest.mark.parametrize("batch", [1, 7, 37, 61])
@pytest.mark.parametrize("kv_heads,group,hd", [(8, 8, 128), (1, 8, 128), (4, 4, 128), (2, 1, 128), (2, 2, 64)])
@pytest.mark.parametrize("num_ctas", [0, 7, 30])
def test_attn_decode(batch, kv_heads, group, hd, num_ctas):
    q_heads = kv_heads * group
    lens = torch.randint(1, 700, (batch,)).tolist()
    lens[0] = 1
    if batch > 2:
        lens[1], lens[2] = 16, 17
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    st = ops.new_status()
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                    num_ctas=num_ctas, status=st)
    ops.check_status(st, "attn_decode")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("chunk_pages", [4, 9, 64])
def test_attn_decode_split_kv(chunk_pages):
    kv_heads, group, hd, batch = 2, 8, 128, 5
    q_heads = kv_heads * group
    lens = [2000, 31, 4096, 640, 1]
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    max_chunks = (256 + chunk_pages - 1) // chunk_pages
    ws = torch.empty(batch * q_heads * max_chunks * (hd + 2), device="cuda", dtype=torch.float32)
    st = ops.new_status()
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                    chunk_pages=chunk_pages, workspace=ws, max_chunks=max_chunks, status=st)
    ops.check_status(st, "attn_decode split")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("M,N,K", [(300, 512, 256), (1000, 1024, 1024), (2048, 1280, 512), (77, 256, 128)])
@pytest.mark.parametrize("tile_m,tile_n,cta_group", [(0, 0, 0), (1, 256, 2), (2, 128, 1), (1, 64, 1)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemm_gated_input_with_flags_already_raised(M, N, K, tile_m, tile_n, cta_group, swiglu):
    """Gated input (row-block flags, tiles walked row block by row block): with every flag at the epoch the
    result is the ungated one bit for bit, for single CTAs, CTA pairs, several M tiles per CTA and SwiGLU;
    ranks beyond gate_nranks are not looked at."""
    if cta_group == 2 and M <= 128:
        pytest.skip("a pair covers two M tiles")
    g = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    w2 = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    blocks = (M + 127) // 128
    flags = torch.zeros(blocks, 8, dtype=torch.int32, device="cuda")
    flags[:, :3] = 7
    flags[:, 0] = 9          # later epochs count as raised
    st = ops.new_status()
    kw = dict(tile_m=tile_m, tile_n=tile_n, cta_group=cta_group, status=st)
    if swiglu:
        want = ops.gemm_swiglu(a, w, w2, **kw)
        got = ops.gemm_swiglu(a, w, w2, gate_flags=flags, gate_epoch=7, gate_nranks=3, **kw)
    else:
        want = ops.gemm(a, w, **kw)
        got = ops.gemm(a, w, gate_flags=flags, gate_epoch=7, gate_nranks=3, **kw)
    ops.check_status(st, "gated gemm")
    assert torch.equal(got, want)


def test_gemm_gated_input_times_out_when_a_flag_never_comes():
    """A row block whose flag is never raised: the producer's bounded wait runs out, the kernel unwinds and
    reports a peer-flag timeout; the context stays usable."""
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    flags = torch.full((2, 8), 3, dtype=torch.int32, device="cuda")
    flags[1, 1] = 2                      # rank 1 never delivers block 1 for epoch 3
    st = ops.new_status()
    ops.gemm(a, w, gate_flags=flags, gate_epoch=3, gate_nranks=2, status=st, tile_m=1, tile_n=128, cta_group=1)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="0x500"):
        ops.check_status(st, "gated gemm")
    assert torch.equal(ops.gemm(a, w), ops.gemm(a, w))


@pytest.mark.parametrize("chunk_pages,max_chunks", [(8, 4), (16, 1), (5, 3)])
def test_attn_decode_split_kv_context_longer_than_the_chunks_cover(chunk_pages, max_chunks):
    """A request with more pages than chunk_pages * max_chunks: the last chunk takes the remaining pages
    (no page is dropped, the merge stays inside the request's workspace slots)."""
    kv_heads, group, hd, batch = 2, 8, 128, 4
    q_heads = kv_heads * group
    lens = [2000, 31, 1500, 640]                 # 125, 2, 94, 40 pages
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    ws = torch.full((batch * q_heads * max_chunks * (hd + 2) + 64,), float("nan"), device="cuda", dtype=torch.float32)
    st = ops.new_status()
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                    chunk_pages=chunk_pages, workspace=ws, max_chunks=max_chunks, status=st)
    ops.check_status(st, "attn_decode split, long context")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)
    assert torch.isnan(ws[-64:]).all()          # nothing was written past the workspace


@pytest.mark.parametrize("kv_heads,group,hd,split", [(1, 8, 128, 0), (8, 8, 128, 0), (2, 2, 64, 0), (2, 8, 128, 9)])
def test_attn_decode_two_pages_in_flight(kv_heads, group, hd, split):
    """The two-stage form of the decode kernel (64 KB of shared memory per CTA instead of 96, for SMs it
    shares with a GEMM CTA and a collective's CTA): same results as the three-stage default."""
    batch = 23
    q_heads = kv_heads * group
    lens = torch.randint(1, 900, (batch,)).tolist()
    lens[0], lens[1], lens[2], lens[3] = 1, 16, 17, 33
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    outs = []
    for stages in (3, 2):
        out = torch.zeros_like(q)
        st = ops.new_status()
        kw = {}
        if split:
            mc = (57 + split - 1) // split
            kw = dict(chunk_pages=split, max_chunks=mc,
                      workspace=torch.empty(batch * q_heads * mc * (hd + 2), device="cuda", dtype=torch.float32))
        ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch,
                        num_ctas=37, status=st, stages=stages, **kw)
        ops.check_status(st, "attn_decode")
        outs.append(out)
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(outs[0], want, atol=1e-2, rtol=2e-2)
    _close(outs[1], want, atol=1e-2, rtol=2e-2)
    with pytest.raises(RuntimeError):
        ops.attn_decode(q, outs[0], pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=0, req_count=batch, stages=4)


def test_attn_decode_request_window():
    """Decode over a sub-range of requests (one attention group of a nano-batch)."""
    kv_heads, group, hd, batch = 1, 8, 128, 20
    q_heads = kv_heads * group
    lens = torch.randint(1, 300, (batch,)).tolist()
    pool, qo, kvp, kvi, last = _make_paged(lens, [1] * batch, kv_heads, hd)
    q = torch.randn(batch, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    ops.attn_decode(q, out, pool, qo, kvp, kvi, last, q_heads=q_heads, req_begin=5, req_count=9)
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads,
                               requests=range(5, 14))
    _close(out, want, atol=1e-2, rtol=2e-2)


def _prefill_items(qo_indptr, group, reqs=None):
    tq = 128 // group
    items = []
    B = len(qo_indptr) - 1
    for b in (reqs if reqs is not None else range(B)):
        t = qo_indptr[b]
        while t < qo_indptr[b + 1]:
            n = min(tq, qo_indptr[b + 1] - t)
            items.append([b, t, n])
            t += n
    return torch.tensor(items, dtype=torch.int32, device="cuda").reshape(-1, 3)


@pytest.mark.parametrize("kv_heads,group,hd", [(1, 8, 128), (8, 8, 128), (4, 4, 128), (2, 1, 128), (2, 2, 64)])
@pytest.mark.parametrize("case", ["short", "long", "chunked", "mixed"])
@pytest.mark.parametrize("impl", ["mma", "tc", "ws"])
def test_attn_prefill(kv_heads, group, hd, case, impl):
    if impl in ("tc", "ws") and hd != 128:
        pytest.skip("the tcgen05 prefill kernel is built for head_dim 128")
    q_heads = kv_heads * group
    if case == "short":
        qo_lens, kv_lens = [1, 5, 16, 17, 33], [1, 5, 16, 17, 33]
    elif case == "long":
        qo_lens, kv_lens = [1024, 300], [1024, 300]
    elif case == "chunked":  # later chunks of a prompt: kv_len > qo_len
        qo_lens, kv_lens = [100, 64, 7], [900, 64 + 512, 2048]
    else:
        qo_lens, kv_lens = [1, 1, 1, 200, 3], [77, 1, 300, 200, 130]
    pool, qo, kvp, kvi, last = _make_paged(kv_lens, qo_lens, kv_heads, hd)
    T = sum(qo_lens)
    q = torch.randn(T, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    items = _prefill_items(qo.tolist(), group)
    st = ops.new_status()
    ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, items, q_heads=q_heads, num_ctas=0 if case != "long" else 11,
                     status=st, impl=impl)
    ops.check_status(st, "attn_prefill")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)


def test_attn_prefill_split_request_across_items():
    """A request whose tokens are covered by items of two nano-batches gives the same rows."""
    kv_heads, group, hd = 1, 8, 128
    q_heads = 8
    pool, qo, kvp, kvi, last = _make_paged([500], [500], kv_heads, hd)
    q = torch.randn(500, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    it_a = torch.tensor([[0, t, min(16, 203 - t)] for t in range(0, 203, 16)], dtype=torch.int32, device="cuda")
    it_b = torch.tensor([[0, t, min(16, 500 - t)] for t in range(203, 500, 16)], dtype=torch.int32, device="cuda")
    ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, it_a, q_heads=q_heads, impl="tc")
    ops.attn_prefill(q, out, pool, qo, kvp, kvi, last, it_b, q_heads=q_heads, impl="mma")
    want = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    _close(out, want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(8, 1, 128), (32, 8, 128), (4, 4, 64)])
@pytest.mark.parametrize("table", [False, True])
def test_rope_append(q_heads, kv_heads, hd, table):
    lens = [40, 1, 17, 300]
    qo_lens = [40, 1, 3, 100]
    pool, qo, kvp, kvi, last = _make_paged(lens, qo_lens, kv_heads, hd)
    pool.zero_()
    T = sum(qo_lens)
    width = (q_heads + 2 * kv_heads) * hd
    qkv = torch.randn(T, width, device="cuda", dtype=torch.bfloat16)
    k_off, v_off, q_off = 0, kv_heads * hd, 2 * kv_heads * hd  # packed K | V | Q
    positions, token_req = [], []
    for b, (l, n) in enumerate(zip(lens, qo_lens)):
        positions += list(range(l - n, l)); token_req += [b] * n
    positions = torch.tensor(positions, dtype=torch.int32, device="cuda")
    token_req = torch.tensor(token_req, dtype=torch.int32, device="cuda")
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    inv = ref.rope_inv_freq(hd, 500000.0, scaling).cuda()
    q_out = torch.empty(T, q_heads * hd, device="cuda", dtype=torch.bfloat16)
    st = ops.new_status()
    cos_sin = None
    if table:   # angles from the per-iteration table instead of computed per token
        cos_sin = ops.rope_table(inv, positions)
        ang = positions.float()[:, None] * inv[None, :]
        _close(cos_sin, torch.stack([ang.cos(), ang.sin()], dim=-1), atol=2e-4, rtol=1e-4)
    ops.rope_append(qkv, q_out, pool, inv, positions, token_req, kvp, kvi, q_heads=q_heads,
                    kv_heads=kv_heads, head_dim=hd, q_off=q_off, k_off=k_off, v_off=v_off, status=st,
                    cos_sin=cos_sin)
    ops.check_status(st, "rope_append")
    pool_ref = torch.zeros_like(pool)
    q_ref = ref.rope_append(qkv, pool_ref, inv, positions.cpu(), token_req.cpu(), kvp.cpu(), kvi.cpu(),
                            q_heads=q_heads, kv_heads=kv_heads, head_dim=hd, q_off=q_off, k_off=k_off,
                            v_off=v_off)
    _close(q_out, q_ref, atol=2e-2, rtol=2e-2)
    _close(pool, pool_ref, atol=2e-2, rtol=2e-2)


def test_kv_move_pages_roundtrip():
    pool = torch.randn(64, 2, 2, 16, 128, device="cuda", dtype=torch.bfloat16)
    ids = torch.tensor([5, 9, 63, 0, 17], dtype=torch.int32, device="cuda")
    staging = torch.empty(5, *pool.shape[1:], device="cuda", dtype=torch.bfloat16)
    ops.kv_move_pages(pool, staging, ids, to_staging=True)
    assert torch.equal(staging, pool[ids.long()])
    pool2 = torch.zeros_like(pool)
    ops.kv_move_pages(pool2, staging, ids, to_staging=False)
    assert torch.equal(pool2[ids.long()], pool[ids.long()])
    assert int((pool2 != 0).sum()) == int((pool[ids.long()] != 0).sum())  # nothing else written


@pytest.mark.parametrize("M,N,K,tile_n,cta_group", [(300, 1024, 512, 0, 0), (1000, 2048, 256, 224, 2), (77, 256, 128, 96, 1),
                                                    (640, 4096, 1024, 256, 2), (129, 1504, 192, 160, 1)])
def test_gemm_reduce_scatter_epilogue_staged_equals_direct(M, N, K, tile_n, cta_group):
    """The reduce-scatter epilogue on one GPU: the slabs of all four owners live in one local buffer, so
    a single launch (rank 1 of 4) can be checked address by address. The staged form (shared memory +
    one bulk copy per row and 128 columns) must leave exactly what the direct form leaves, in the same
    places: row i at slab[owner i % 4][rank 1][i // 4], nothing outside, the ready flag of rank 1 raised
    on every owner."""
    import ctypes

    from nanoflow_b200 import ops
    from nanoflow_b200.ops import GemmParams

    world, rank = 4, 1
    g = torch.Generator(device="cpu").manual_seed(5)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    cap = (M + world - 1) // world
    region = ((world * cap * N * 2 + 255) // 256 + 2) * 256          # per-owner "heap": flags (256 B) + slabs + guard
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for staged in (0, 1):
        heap = torch.full((world * region,), 0x7F, dtype=torch.uint8, device="cuda")
        for r in range(world):
            heap[r * region:r * region + 256] = 0                       # flag blocks start cleared
        p = GemmParams()
        p.A, p.B, p.D = a.data_ptr(), w.data_ptr(), 0
        p.lda, p.ldb, p.ldd = K, K, N
        p.M, p.N, p.K, p.epilogue = M, N, K, 2
        p.tile_n, p.cta_group = tile_n, cta_group
        for r in range(world):
            p.rs_heap[r] = heap.data_ptr() + r * region
        p.rs_rank, p.rs_nranks, p.rs_rows_cap = rank, world, cap
        p.rs_slab_off, p.rs_flag_off, p.rs_epoch = 256, 0, 7
        p.rs_staged = staged
        p.status = status.data_ptr()
        rc = ops.lib().nfk_gemm_bf16(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, rc
        torch.cuda.synchronize()
        ops.check_status(status, "gemm")
        outs.append(heap)
    direct, staged = outs
    assert torch.equal(direct, staged)
    want = (a.float() @ w.float().t())
    for owner in range(world):
        base = owner * region
        flags = staged[base:base + 256].view(torch.int32)
        assert flags[rank].item() == 7 and flags[16].item() == 0 and int((flags != 0).sum()) == 1
        slabs = staged[base + 256:base + 256 + world * cap * N * 2].view(torch.bfloat16).view(world, cap, N)
        rows = torch.arange(owner, M, world, device="cuda")
        got = slabs[rank, :rows.numel()].float()
        assert torch.allclose(got, want[rows], atol=4e-2 * (K / 64) ** 0.5, rtol=2e-2)
        untouched = torch.ones(world, cap, dtype=torch.bool, device="cuda")
        untouched[rank, :rows.numel()] = False
        assert bool((slabs.view(torch.int16)[untouched] == 0x7F7F).all())
        assert bool((staged[base + 256 + world * cap * N * 2:base + region] == 0x7F).all())


def test_strided_copy_op_moves_every_nth_row():
    """nfk_memcpy2d_p (the op that delivers a rank's normed rows to a peer through the copy engines):
    rows r, r + n, r + 2n, ... of one buffer land in the same rows of another, nothing else is touched."""
    from ctypes import byref, c_void_p

    from nanoflow_b200.runtime.graph import Memcpy2DParams

    rows, cols, n, r = 37, 512, 8, 3
    src = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    dst = torch.full_like(src, -1.0)
    own = (rows - r + n - 1) // n
    p = Memcpy2DParams()
    row_bytes = cols * 2
    p.dst, p.src = dst.data_ptr() + r * row_bytes, src.data_ptr() + r * row_bytes
    p.dpitch = p.spitch = n * row_bytes
    p.width, p.height = row_bytes, own
    rc = ops.lib().nfk_memcpy2d_p(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    mine = torch.arange(r, rows, n, device="cuda")
    assert torch.equal(dst[mine], src[mine])
    others = torch.tensor([i for i in range(rows) if i % n != r], device="cuda")
    assert bool((dst[others] == -1.0).all())
    p.height = 0
    assert ops.lib().nfk_memcpy2d_p(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
