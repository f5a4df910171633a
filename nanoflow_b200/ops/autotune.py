"""Measured choice of the GEMM kernel shape for the shapes an engine actually runs.

The launcher's cost model (csrc/kernels/gemm.cu, ``choose_shape``) ranks tile shapes from a few
constants; on a power-capped GPU those constants move with the clock the part settles at. Before an
engine builds its op graph it therefore times a short list of candidates per (op, nano-batch size)
on its own buffers and weights and pins the fastest: tile width, M tiles per CTA, CTA pairs, split-K,
stream-K tail. Successive runs use the weights of different layers, so a weight matrix that fits in
L2 is still read from HBM as it is in a real iteration.

The reference picks a CUTLASS configuration per operator from offline profiling: genGEMM.py
generates the candidate instantiations (pipeline/src/generate-gemm/genGEMM.py,
pipeline/include/gemmFactory.cuh) and each pipeline class carries the chosen names in its
``gemmConfig`` table (pipeline/include/pipeline.h:69, 189, 267, 336, 415). This is the on-line
equivalent.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from . import gemm, gemm_swiglu

KEYS = ("tile_m", "tile_n", "cta_group", "split_k", "stream_k")
AUTO: Dict[str, int] = dict(tile_m=0, tile_n=0, cta_group=0, split_k=0, stream_k=0)


def candidates(M: int, N: int, K: int, swiglu: bool) -> List[Dict[str, int]]:
    """Shapes worth timing for an M x N x K product (N = output columns; SwiGLU tiles hold a gate and
    an up half, so their width counts twice)."""
    m_tiles = (M + 127) // 128
    num_kb = (K + 63) // 64
    out: List[Dict[str, int]] = [dict(AUTO)]

    def add(tm, tn, cg, sk=1, tail=2):
        c = dict(tile_m=tm, tile_n=tn, cta_group=cg, split_k=sk, stream_k=tail)
        if c not in out:
            out.append(c)

    widths = (256, 224, 192) if swiglu else (256, 224, 192, 128)
    splits = (1,) if swiglu else tuple(s for s in (1, 2, 3, 4) if num_kb // s >= 8)
    for tn in widths:
        for tail in (2, 1):
            add(1, tn, 1, 1, tail)
            if m_tiles >= 2:
                add(1, tn, 2, 1, tail)
    if not swiglu and m_tiles >= 2:
        # pair tiles wider than one MMA instruction: fewer, fatter tiles (a wave of 64 tiles of 256 x 320 where
        # 256-wide ones make 80 on 74 pairs), each weight byte fetched for 256 rows and each activation byte
        # for 320 or more columns
        for tn in (320, 384, 512):
            if N >= tn:
                add(1, tn, 2, 1, 2)
    if m_tiles <= 4:
        for tm, tn in ((2, 256), (2, 224), (2, 128), (4, 128)):
            if m_tiles > tm // 2:
                for tail in (2, 1):
                    add(tm, tn, 1, 1, tail)
    for sk in splits:
        if sk == 1:
            continue
        add(1, 256, 1, sk)
        if m_tiles >= 2:
            add(1, 256, 2, sk)
        if m_tiles <= 4 and m_tiles > 1:
            add(2, 256, 1, sk)
    return out


def tune_gemm(a: torch.Tensor, weights: Sequence[torch.Tensor], out: torch.Tensor, *,
              weights_up: Optional[Sequence[torch.Tensor]] = None, residual: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, num_ctas: int = 0, workspace: Optional[torch.Tensor] = None,
              smem_budget_kb: int = 0, iters: int = 4, passes: int = 2) -> Dict[str, object]:
    """Time every candidate on ``a @ weights[i]^T`` (cycling through ``weights``) and return
    ``{"best": kwargs, "us": best time, "auto_us": time of the cost model's own choice, "table": [...]}``.
    Candidates the launcher rejects (shape not built, workspace too small) are skipped."""
    M, K = a.shape
    N = weights[0].shape[0]
    swiglu = weights_up is not None
    cands = candidates(M, N, K, swiglu)
    best_us = [float("inf")] * len(cands)
    layer = 0

    def run(c, i):
        w = weights[i % len(weights)]
        if swiglu:
            gemm_swiglu(a, w, weights_up[i % len(weights)], out=out, num_ctas=num_ctas, workspace=workspace,
                        smem_budget_kb=smem_budget_kb, tile_m=c["tile_m"], tile_n=c["tile_n"],
                        cta_group=c["cta_group"], stream_k=c["stream_k"])
        else:
            gemm(a, w, out=out, residual=residual, bias=bias, num_ctas=num_ctas, workspace=workspace,
                 smem_budget_kb=smem_budget_kb, **c)

    for _ in range(passes):
        for ci, c in enumerate(cands):
            if best_us[ci] < 0:
                continue
            try:
                run(c, layer)
            except RuntimeError:
                best_us[ci] = -1.0           # not available for this shape
                continue
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(iters):
                run(c, layer + 1 + i)
            e1.record()
            e1.synchronize()
            layer += iters + 1
            best_us[ci] = min(best_us[ci], e0.elapsed_time(e1) * 1e3 / iters)
    table = [dict(c, us=round(t, 2)) for c, t in zip(cands, best_us) if t >= 0]
    table.sort(key=lambda r: r["us"])
    auto_us = next(r["us"] for r in table if all(r[k] == 0 for k in KEYS))
    top = table[0]
    # keep the cost model's choice unless a pinned shape is clearly faster (timing noise is a few %)
    best = {k: top[k] for k in KEYS} if top["us"] < 0.97 * auto_us else dict(AUTO)
    return dict(best=best, us=top["us"], auto_us=auto_us, table=table)
