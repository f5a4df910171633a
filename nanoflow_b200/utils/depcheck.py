"""Static race check of an op graph.

Every op is annotated (by the kernel it calls) with the device buffers it reads and writes, as byte
ranges taken from its parameter block. Two ops conflict when one writes a range the other reads or
writes; the check demands a happens-before edge (explicit dependency or stream order, transitively)
between every conflicting pair. The reference relies on hand-placed event waits for this
(pipeline/src/pipeline.cu:628-733) and has no checker.

Ranges are conservative: a GEMM is taken to touch ``rows_cap`` rows of its operands (the static
capacity of its nano-batch), not the dynamic row count.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from ..runtime.graph import OpGraph

Range = Tuple[int, int]   # [begin, end) device addresses


def _overlap(a: Range, b: Range) -> bool:
    return a[0] < b[1] and b[0] < a[1]


def conflicts(reads_a: List[Range], writes_a: List[Range], reads_b: List[Range], writes_b: List[Range]) -> bool:
    for w in writes_a:
        if any(_overlap(w, r) for r in reads_b) or any(_overlap(w, x) for x in writes_b):
            return True
    for w in writes_b:
        if any(_overlap(w, r) for r in reads_a):
            return True
    return False


def check(graph: OpGraph, access: Dict[int, Tuple[List[Range], List[Range]]]) -> List[Tuple[int, int]]:
    """``access[i] = (reads, writes)`` for op i. Returns conflicting pairs without an ordering."""
    hb = graph.happens_before()
    bad = []
    idx = sorted(access)
    for ai, i in enumerate(idx):
        ri, wi = access[i]
        for j in idx[ai + 1:]:
            rj, wj = access[j]
            if not conflicts(ri, wi, rj, wj):
                continue
            if i in hb[j] or j in hb[i]:
                continue
            bad.append((i, j))
    return bad


# ---- access extraction from parameter blocks ------------------------------------------------------
def graph_access(graph: OpGraph, nano_starts: List[int], nano_sizes: List[int], heap_base: int = 0,
                 kv_pool_bytes: int = 0, peer_bases: List[int] = ()) -> Dict[int, Tuple[List[Range], List[Range]]]:
    """Read / write byte ranges of every op, from its parameter block. Row counts that are dynamic
    (symbols) are replaced by the capacity of the op's nano-batch (or ``sum(nano_sizes)``).

    ``peer_bases``: where the ranks' symmetric heaps are mapped. A strided copy into a peer's heap stands
    for the copy that the peer issues into this rank's heap at the same moment, so its target is taken at the
    same offset of this rank's heap."""
    from ..parallel.collectives import AllGatherParams, AllReduceParams
    from ..runtime import graph as G

    total = sum(nano_sizes)
    out: Dict[int, Tuple[List[Range], List[Range]]] = {}
    # KV pages belong to requests, and a request's tokens of one iteration sit in one nano-batch (a
    # decode token) or in consecutive ones (a prompt chunk that straddles a cut). The RoPE / append op
    # of nano-batch k therefore writes pages that only the attention of nano-batch k, and the prefill
    # attention of later nano-batches, read. The check stands for that with one slice of the pool's
    # address range per nano-batch.
    nn = max(1, len(nano_sizes))

    def pool_slice(base: int, k0: int, k1: int) -> Range:
        sub = kv_pool_bytes // nn
        return (base + k0 * sub, base + (k1 + 1) * sub if k1 + 1 < nn else base + kv_pool_bytes)

    def rng(ptr, rows, ld_elems, cols, esz=2):
        if not ptr or rows <= 0:
            return None
        return (int(ptr), int(ptr) + ((rows - 1) * ld_elems + cols) * esz)

    for i, op in enumerate(graph.ops):
        p = op.params
        cap = nano_sizes[op.nano] if op.nano >= 0 else total
        reads: List[Range] = []
        writes: List[Range] = []
        add = lambda lst, r: lst.append(r) if r is not None else None
        if isinstance(p, G.GemmParams):
            rows = cap if op.nano >= 0 else total
            add(reads, rng(p.A, rows, p.lda, p.K))
            add(reads, rng(p.B, p.N, p.ldb, p.K))
            add(reads, rng(p.B2, p.N, p.ldb, p.K))
            add(reads, rng(p.C, rows, p.ldc, p.N))
            if p.epilogue == 2:      # reduce-scatter epilogue: pushes into the slabs (this rank's image of them)
                base = (p.rs_heap[p.rs_rank] or 0) + p.rs_slab_off
                add(writes, (base, base + p.rs_nranks * p.rs_rows_cap * p.N * 2))
            else:
                add(writes, rng(p.D, rows, p.ldd, p.N))
            if p.workspace:
                add(writes, (int(p.workspace), int(p.workspace) + int(p.workspace_bytes)))
            if p.norm_w:
                add(writes, rng(p.norm_out, rows, p.norm_ld, p.N))
        elif isinstance(p, G.NormParams):
            add(reads, rng(p.x, cap, p.cols, p.cols))
            add(writes, rng(p.out, cap, p.cols, p.cols))
            if p.resid:
                add(writes, rng(p.resid, cap, p.cols, p.cols))
        elif isinstance(p, G.RopeAppendParams):
            width = (p.q_heads + 2 * p.kv_heads) * p.head_dim
            add(reads, rng(p.qkv, cap, p.ld_qkv, width))
            add(writes, rng(p.q_out, cap, p.q_heads * p.head_dim, p.q_heads * p.head_dim))
            add(reads, rng(p.cos_sin, cap, p.head_dim, p.head_dim, 4))
            if kv_pool_bytes:
                k = op.nano if op.nano >= 0 else 0
                add(writes, pool_slice(int(p.kv_pool), k, k) if op.nano >= 0 else
                    (int(p.kv_pool), int(p.kv_pool) + kv_pool_bytes))
        elif isinstance(p, G.RopeTableParams):
            add(writes, rng(p.cos_sin, total, 2 * p.half, 2 * p.half, 4))
        elif isinstance(p, G.AttnParams):
            # q / out rows of the whole dense batch are addressable; the op touches its nano-batch's rows
            r0 = nano_starts[op.nano] if op.nano >= 0 else 0
            w = p.q_heads * p.head_dim
            add(reads, rng(p.q + r0 * w * 2, cap, w, w))
            # A nano-batch holds its decode tokens first and its prompt tokens after them, and the two
            # kernels write only their own tokens' rows. The boundary moves every iteration; the check
            # stands for it with the middle of the nano-batch, which keeps the two writers disjoint
            # from each other and both in conflict with every reader of the rows.
            half = cap // 2
            if op.kernel == "nfk_attn_decode":
                add(writes, rng(p.out + r0 * w * 2, half, w, w))
            else:
                add(writes, rng(p.out + (r0 + half) * w * 2, cap - half, w, w))
            if kv_pool_bytes:
                if op.nano < 0:
                    add(reads, (int(p.kv_pool), int(p.kv_pool) + kv_pool_bytes))
                elif op.kernel == "nfk_attn_decode":
                    add(reads, pool_slice(int(p.kv_pool), op.nano, op.nano))
                else:       # prefill: its own nano-batch's appends and, for a straddling prompt, earlier ones'
                    add(reads, pool_slice(int(p.kv_pool), 0, op.nano))
        elif isinstance(p, AllReduceParams):
            base = heap_base + p.buf_off
            if p.src_mode == 1:
                buf = (base, base + p.ctx.nranks * p.slab_rows * p.ld * 2)
            else:
                buf = rng(base, cap, p.ld, p.cols)
            add(reads, buf)
            if p.push_sum:
                add(writes, buf)
            add(reads, rng(p.resid, cap, p.resid_ld, p.cols))
            add(writes, rng(p.sum_out, cap, p.sum_ld, p.cols))
            if p.norm_w:
                add(writes, rng(heap_base + p.norm_out_off, cap, p.norm_ld, p.cols))
        elif isinstance(p, G.Memcpy2DParams):
            rows = cap
            if any(f == "height" and sym.endswith("_own_rows") for f, sym in op.dyn) and peer_bases:
                rows = (cap + len(peer_bases) - 1) // len(peer_bases)      # every tp-th row of the nano-batch
            span = lambda ptr, pitch: (int(ptr), int(ptr) + (max(rows, 1) - 1) * int(pitch) + int(p.width))
            add(reads, span(p.src, p.spitch))
            dst = int(p.dst)
            below = [b for b in peer_bases if b and b <= dst]
            if below and heap_base:
                dst = heap_base + (dst - max(below))
            add(writes, span(dst, p.dpitch))
        elif isinstance(p, G.GatherParams):
            add(reads, rng(p.inp, p.in_rows, p.ld_in, p.cols))
            add(writes, rng(p.out, total, p.cols, p.cols))
        elif isinstance(p, G.EmbeddingParams):
            add(writes, rng(p.out, total, p.hidden, p.hidden))
        else:
            continue
        out[i] = (reads, writes)
    return out
