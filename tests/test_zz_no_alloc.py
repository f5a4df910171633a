"""Allocation-free split-KV decode attention (``nfk_attn_decode_static``), called through its
exported C symbol, against the regular entry point that takes a caller-provided workspace.

The static variant exists for callers that cannot allocate device memory when they need attention
(for instance an engine whose KV pool already took all free memory); its scratch is a fixed 8 MiB
array inside the library. Two calls in a row must both match, since they share that array.
"""
import ctypes
from ctypes import byref, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

from nanoflow_b200 import ops


def _problem(batch, kv_heads, group, hd, lens, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    page = 16
    npages = [(l + page - 1) // page for l in lens]
    total = sum(npages) + 3
    perm = torch.randperm(total, generator=g)
    kv_indptr = [0]
    for n in npages:
        kv_indptr.append(kv_indptr[-1] + n)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    pool = torch.randn(total, 2, kv_heads, page, hd, generator=g).bfloat16().cuda()
    q = torch.randn(batch, kv_heads * group * hd, generator=g).bfloat16().cuda()
    return (pool, q, dev(list(range(batch + 1))), dev(kv_indptr), perm[:kv_indptr[-1]].int().cuda(),
            dev([(l - 1) % page + 1 for l in lens]))


def _params(q, out, pool, qo, kvp, kvi, last, q_heads, chunk_pages, max_chunks, workspace):
    p = ops._attn_common(q, out, pool, qo, kvp, kvi, last, q_heads, None, 0, None)
    p.req_begin, p.req_count = 0, q.shape[0]
    p.chunk_pages, p.max_chunks = chunk_pages, max_chunks
    p.workspace = c_void_p(0 if workspace is None else workspace.data_ptr())
    return p


def test_static_scratch_decode_matches_workspace_decode_twice():
    lib = ops.lib()
    fn = lib.nfk_attn_decode_static
    fn.restype = ctypes.c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (lens, seed) in enumerate([([2000, 31, 4096, 640, 1, 777], 1), ([4096, 4096, 100, 16, 3000, 2049], 2)]):
        kv_heads, group, hd = 2, 8, 128
        q_heads = kv_heads * group
        batch = len(lens)
        pool, q, qo, kvp, kvi, last = _problem(batch, kv_heads, group, hd, lens, seed)
        chunk_pages, max_chunks = 16, 16
        ws = torch.empty(batch * q_heads * max_chunks * (hd + 2), device="cuda", dtype=torch.float32)
        want = torch.zeros_like(q)
        rc = lib.nfk_attn_decode(byref(_params(q, want, pool, qo, kvp, kvi, last, q_heads, chunk_pages,
                                               max_chunks, ws)), stream)
        assert rc == 0
        got = torch.zeros_like(q)
        rc = fn(byref(_params(q, got, pool, qo, kvp, kvi, last, q_heads, chunk_pages, max_chunks, None)), stream)
        assert rc == 0, f"call {call}: nfk_attn_decode_static returned {rc}"
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        err = (got.float() - want.float()).abs()
        assert bool((err <= 1e-2 + 2e-2 * want.float().abs()).all()), f"call {call}: max err {err.max().item()}"
        # and both agree with the fp32 restatement
        from nanoflow_b200.ops import reference as ref
        oracle = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
        assert bool(((got.float() - oracle).abs() <= 1e-2 + 2e-2 * oracle.abs()).all())


def test_static_scratch_context_longer_than_the_chunks_cover():
    """More pages than chunk_pages * max_chunks: the last chunk absorbs the rest, as in the workspace entry."""
    lib = ops.lib()
    fn = lib.nfk_attn_decode_static
    fn.restype = ctypes.c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    kv_heads, group, hd = 2, 8, 128
    q_heads = kv_heads * group
    lens = [2000, 31, 1500]
    pool, q, qo, kvp, kvi, last = _problem(len(lens), kv_heads, group, hd, lens, 5)
    got = torch.zeros_like(q)
    rc = fn(byref(_params(q, got, pool, qo, kvp, kvi, last, q_heads, 8, 4, None)), stream)
    assert rc == 0
    torch.cuda.synchronize()
    from nanoflow_b200.ops import reference as ref
    oracle = ref.paged_attention(q, pool, qo.cpu(), kvp.cpu(), kvi, last.cpu(), q_heads=q_heads)
    assert bool(((got.float() - oracle).abs() <= 1e-2 + 2e-2 * oracle.abs()).all())


def test_static_scratch_rejects_oversized_request():
    lib = ops.lib()
    fn = lib.nfk_attn_decode_static
    fn.restype = ctypes.c_int
    kv_heads, group, hd, batch = 8, 8, 128, 64
    lens = [64] * batch
    pool, q, qo, kvp, kvi, last = _problem(batch, kv_heads, group, hd, lens, 3)
    out = torch.zeros_like(q)
    # 64 requests x 64 heads x 16 chunks x 130 floats = 8.5 M floats > 2 M floats of fixed scratch
    rc = fn(byref(_params(q, out, pool, qo, kvp, kvi, last, kv_heads * group, 2, 16, None)),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 1
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0      # nothing was launched
    # without a split no scratch is needed and the same shapes are accepted
    rc = fn(byref(_params(q, out, pool, qo, kvp, kvi, last, kv_heads * group, 0, 1, None)),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
