"""Builds the per-iteration op graph of a Llama-family decoder from the config.

One graph covers the whole iteration: token-id feedback + embedding, ``run_layers`` decoder layers
over every nano-batch, and the sampling epilogue (gather last-token rows, final norm, vocab-sharded
LM head, arg-max, cross-rank combine). Nano-batches own fixed row ranges of the activation buffers;
their token counts are symbols, so the graph is built once.

Pipeline variants (the reference's ``PipelineType``s, pipeline/include/pipeline.h:53-468,
selected by ``serve_configs.pipeline_type``):

* ``NON_OVERLAP*``   one nano-batch, every op on one stream.
* ``NANOBATCH*``     nano-batches, still one stream (isolates the cost of splitting the batch).
* ``PLLM / LOCAL / KQVBIAS / PLLM_OFFLOAD``  nano-batches, ops spread over the gemm / attn / net /
  other / copy streams with event dependencies, issue order software-pipelined so that the
  attention of one nano-batch runs next to the GEMMs of the other (reference schedule:
  pipeline/src/pipeline.cu:628-733 for TP, pipeline/src/pipeline_local.cu:353-431 for one GPU), and
  CTA budgets taken from ``pipeline_configs.sm_budget``.

Tensor parallel layout per layer: QKV (K|V|Q packed, N-split) -> RoPE/append -> attention (head
parallel) -> O (K-split partial products) -> reduce-scatter + residual + RMSNorm + all-gather in one
collective -> gate/up (N-split, SwiGLU epilogue) -> down (K-split) -> the same collective with the
next layer's attention norm. The residual stream stays sharded by row owner between layers; only
normed activations cross NVLink on the gather side.
"""
from __future__ import annotations

from ctypes import c_void_p
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from .. import ops as _ops
from ..config import EngineConfig, ModelConfig
from ..models.llama import RankWeights
from .graph import (ArgmaxCombineParams, ArgmaxParams, AttnParams, EmbeddingParams, GatherParams, GemmParams, RopeTableParams,
                    KvMoveParams, MemcpyParams, NormParams, OpGraph, RopeAppendParams)


def _ptr(t: Optional[torch.Tensor], row: int = 0) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr() + row * t.stride(0) * t.element_size())


@dataclass
class Buffers:
    """Device tensors an iteration reads and writes (allocated once by the engine)."""
    x: List[torch.Tensor]            # residual stream, two buffers [T, hidden]
    h: torch.Tensor                  # normed activations [T, hidden]
    qkv: torch.Tensor                # [T, qkv_local]
    q_rot: torch.Tensor              # [T, q_local]
    attn_out: torch.Tensor           # [T, q_local]
    act: torch.Tensor                # [T, ffn_local]
    sample_h: torch.Tensor           # [B, hidden]
    sample_hn: torch.Tensor          # [B, hidden]
    logits: torch.Tensor             # [B, vocab_local]
    cand_val: torch.Tensor           # [tp, B] fp32 (symmetric under TP)
    cand_idx: torch.Tensor           # [tp, B] int32
    sampled: torch.Tensor            # [B] int32 tokens of the last iteration (device feedback source)
    kv_pool: List[torch.Tensor]      # per layer [pages, 2, kv_heads_local, page, head_dim]
    inv_freq: torch.Tensor           # [head_dim/2] fp32
    status: torch.Tensor             # [1] int32
    decode_ws: Optional[torch.Tensor]  # split-KV workspace (fp32)
    meta: Dict[str, torch.Tensor]    # int32 views into the metadata block (see engine.MetaLayout)
    nano_items: List[torch.Tensor]   # per nano-batch [cap,3] int32 views
    gemm_ws: Optional[torch.Tensor] = None   # split-K partial sums (fp32); all GEMMs share one stream
    attn_full: Optional[torch.Tensor] = None  # [T, q_size] symmetric: all ranks' attention outputs side by side
                                              # (only with nano-batches whose O projection takes the all-gather form)
    rope_table: Optional[torch.Tensor] = None  # [T, head_dim/2, 2] fp32 angles of the iteration's tokens


class CollectiveHooks:
    """Adds the tensor-parallel collectives to the graph. The TP1 default adds nothing."""
    tp = 1

    def all_reduce(self, g: OpGraph, name: str, buf: torch.Tensor, row0: int, rows_sym: str, cols: int,
                   deps, layer: int, nano: int, stream: str = "net", norm_w=None, norm_out=None,
                   eps: float = 1e-5, status=None, num_ctas: int = 0, resid=None, sum_out=None,
                   push_sum: bool = True):
        """Returns (op index or None, whether the RMSNorm was fused into the collective)."""
        return None, False

    def all_gather_candidates(self, g: OpGraph, bufs: Buffers, rows_sym: str, deps) -> Optional[int]:
        return None

    def all_gather_columns(self, g: OpGraph, name: str, src: torch.Tensor, dst: torch.Tensor, row0: int,
                           rows_sym: str, deps, layer: int, nano: int, stream: str = "net", status=None):
        return None


@dataclass
class IoSpec:
    """Where the iteration's host<->device copies go: the metadata block and the sampled tokens."""
    meta_dev: torch.Tensor      # int32 block on the device
    fixed_words: int            # words [0, fixed_words) are copied every iteration
    kv_off_words: int           # start of the kv_indices array (a prefix of it is copied)
    offload_staging: Optional[torch.Tensor] = None   # device [cap, page_elems] gather target (KV offload)
    offload_pages: Optional[torch.Tensor] = None     # int32 view: page ids of requests retired this iteration


# Shared memory a GEMM CTA may take when a collective's CTAs are meant to run beside it on the same
# SM: the SM has 228 KB and every resident CTA reserves 1 KB plus its own static allocation.
GEMM_SMEM_KB_SHARED_SM = 200
# ... and when a decode-attention CTA (96 KB) is meant to sit on the same SM as well (attn_overlap).
GEMM_SMEM_KB_BESIDE_ATTENTION = 130


def default_comm_ctas(tp: int, in_switch: bool) -> int:
    """CTAs of a collective that runs beside other kernels (overlapped pipelines). A collective's CTAs slow
    whatever shares their SMs (eight GPUs, in-switch all-reduce: 161.0 / 161.1 / 164.6 / 166.3 ms per
    iteration with 16 / 32 / 96 / 148 CTAs), while the in-switch all-reduce alone is as fast with 32 CTAs as
    with 96 at eight ranks (a rank then owns 512 of a nano-batch's 4096 rows, 16 per CTA). So: about 16 owned
    rows per CTA for the in-switch form; the peer-load form needs its loads in flight and keeps 96."""
    if not in_switch:
        return 96
    return max(16, min(96, 256 // max(1, tp)))


def gemm_smem_budget_kb(eng: EngineConfig, tp: int) -> int:
    """Shared memory a GEMM CTA may take in this pipeline (0 = all of it)."""
    if not (eng.overlap and tp > 1):
        return 0
    return GEMM_SMEM_KB_BESIDE_ATTENTION if eng.attn_overlap else GEMM_SMEM_KB_SHARED_SM


def build_graph(model: ModelConfig, eng: EngineConfig, w: RankWeights, bufs: Buffers,
                coll: Optional[CollectiveHooks] = None, io: Optional[IoSpec] = None) -> OpGraph:
    coll = coll or CollectiveHooks()
    tp = w.tp
    g = OpGraph()
    overlap = eng.overlap
    sizes = eng.resolved_nanobatches()
    starts = [sum(sizes[:k]) for k in range(len(sizes))]
    nn = len(sizes)
    hd, hidden = model.head_dim, model.hidden_size
    st = bufs.status
    budget = eng.sm_budget if overlap else {}
    # Stream chooser. Collectives always get the net stream in overlap mode: their CTAs need no
    # shared memory and co-reside with GEMM CTAs. Attention CTAs cannot share an SM with a GEMM CTA
    # (shared memory), so under tensor parallelism they stay in line with the GEMMs; on one GPU
    # (LOCAL pipelines) they get their own stream and fill SMs as GEMM CTAs retire.
    if not overlap:
        S = lambda cls: "gemm"
    elif tp > 1 and eng.attn_overlap:
        # Decode attention (memory-bound) on its own stream under the GEMMs (compute-bound) of the other
        # nano-batches: one decode CTA (96 KB) per SM fits beside a GEMM CTA that keeps to 130 KB of shared
        # memory (with the 1 KB reserved per CTA that is the whole SM, so a collective's CTA joins only
        # once the decode CTA has left). The O projections are issued after all nano-batches' front-ends
        # so that the compute stream does not wait behind an attention kernel.
        S = lambda cls: cls if cls in ("net", "attn") else "gemm"
    elif tp > 1:
        S = lambda cls: "net" if cls == "net" else "gemm"
    else:
        S = lambda cls: cls
    # Prefill and decode attention of one nano-batch touch different requests. The decode kernel's work
    # items rarely fill its last round of CTAs, so the prefill kernel, on a stream of its own, runs in
    # the SMs that round leaves idle. The O projection, next on the GEMM stream, waits for both, so no
    # GEMM is ever queued beside the pair.
    prefill_stream = "attn2" if eng.prefill_beside_decode else S("attn")
    if overlap and tp > 1 and eng.attn_overlap and eng.cross_layer_pipeline:
        # Skewed schedule (below): only the decode kernel is small enough to sit on an SM beside a GEMM CTA;
        # a prefill CTA (97 KB) would have to wait for a GEMM CTA to leave and then hold the next
        # GEMM's CTA off that SM, so prefill attention stays in line on the compute stream.
        prefill_stream = "gemm"
    # Collectives of one nano-batch never depend on those of another, and each is bound by the latency of
    # its peer loads rather than by the links; with two network streams the collective of an odd
    # nano-batch starts when its GEMM is done instead of queueing behind the previous one.
    net_of = lambda k: "net2" if (eng.net_streams > 1 and S("net") == "net" and k % 2 == 1) else S("net")

    T_all = g.symbol("T")
    n_sample = g.symbol("n_sample")
    nb_T = [g.symbol(f"nb{k}_T") for k in range(nn)]
    nb_dec0 = [g.symbol(f"nb{k}_dec_begin") for k in range(nn)]
    nb_decn = [g.symbol(f"nb{k}_dec_count") for k in range(nn)]
    nb_items = [g.symbol(f"nb{k}_items") for k in range(nn)]
    chunk_pages = g.symbol("decode_chunk_pages")
    max_chunks = g.symbol("decode_max_chunks")

    m = bufs.meta
    # ---- prologue: ids (device feedback) + embedding into residual buffer 0 ------------------------
    ep = EmbeddingParams(out=_ptr(bufs.x[0]), table=_ptr(w.embed), host_ids=_ptr(m["host_ids"]),
                         feedback_src=_ptr(m["feedback_src"]), prev_tokens=_ptr(bufs.sampled),
                         ids_out=c_void_p(0), n_tokens=0, hidden=hidden, vocab=model.vocab_size, status=_ptr(st))
    pre = []
    if io is not None:
        # pinned host -> device metadata copies; the source slot rotates, so the pointers are symbols
        c1 = MemcpyParams(dst=_ptr(io.meta_dev), src=c_void_p(0), elem_bytes=4, count=io.fixed_words)
        pre.append(g.add("meta_h2d", c1, S("other"), dyn=[("src", g.symbol("meta_src"))]))
        c2 = MemcpyParams(dst=c_void_p(io.meta_dev.data_ptr() + 4 * io.kv_off_words), src=c_void_p(0),
                          elem_bytes=4, count=0)
        pre.append(g.add("kv_indices_h2d", c2, S("other"),
                         dyn=[("src", g.symbol("kv_src")), ("count", g.symbol("kv_words"))]))
    if bufs.rope_table is not None:
        # cos / sin of every token's rotary angles, once per iteration for all layers
        tp_ = RopeTableParams()
        tp_.cos_sin, tp_.inv_freq, tp_.positions = _ptr(bufs.rope_table), _ptr(bufs.inv_freq), _ptr(m["positions"])
        tp_.T, tp_.half = 0, hd // 2
        pre.append(g.add("rope_table", tp_, S("other"), deps=list(pre), dyn=[("T", T_all)]))
    emb = g.add("embedding", ep, S("other"), deps=pre, dyn=[("n_tokens", T_all)])

    last_x_writer: List[Optional[int]] = [emb] * nn     # op that last wrote nano-batch k's residual rows
    prev_attn: List[Optional[int]] = [None] * nn
    cur = 0                                             # which residual buffer holds x

    def gemm(name, a, wt, out, k, *, residual=None, beta=1.0, bias=None, swiglu_up=None, deps=(), layer=-1,
             tile_key=None, rs=None, norm=None, gate=None):
        p = GemmParams()
        r0 = starts[k]
        p.A, p.B, p.D = _ptr(a, r0), _ptr(wt), (_ptr(out, r0) if out is not None else c_void_p(0))
        p.B2 = _ptr(swiglu_up)
        p.C, p.bias = _ptr(residual, r0) if residual is not None else c_void_p(0), _ptr(bias)
        p.lda, p.ldb, p.ldd = a.stride(0), wt.stride(0), (out.stride(0) if out is not None else wt.shape[0])
        p.ldc = residual.stride(0) if residual is not None else 0
        p.beta, p.M, p.N, p.K = beta, 0, wt.shape[0], wt.shape[1]
        p.epilogue = 1 if swiglu_up is not None else 0
        if norm is not None:
            # RMSNorm of the result rows for the next GEMM, from the same call (see kernels.h)
            p.norm_w, p.norm_out = _ptr(norm[0]), _ptr(norm[1], r0)
            p.norm_ld, p.norm_eps = norm[1].stride(0), model.rms_norm_eps
        dyn = [("M", nb_T[k])]
        if rs is not None:
            # fused GEMM -> reduce-scatter: the epilogue pushes partial rows to their owners' slabs
            p.epilogue = 2
            for r, base in enumerate(rs["heap"]):
                p.rs_heap[r] = base
            p.rs_rank, p.rs_nranks, p.rs_rows_cap = rs["rank"], rs["nranks"], rs["rows_cap"]
            p.rs_slab_off, p.rs_flag_off = rs["slab_off"], rs["flag_off"]
            p.rs_staged = 1 if eng.gemm_rs_staged else 0
            dyn.append(("rs_epoch", g.symbol("epoch")))
        key = tile_key or name.split(".")[-1]
        p.tile_n = eng.gemm_tile_n.get(key, 0)
        gated = ()
        if gate is not None:
            # rows of `a` arrive block by block from the collective `gate["op"]`: launch with it, wait per M tile
            p.gate_flags, p.gate_nranks = gate["flags"], gate["nranks"]
            dyn.append(("gate_epoch", g.symbol("epoch")))
            gated = [gate["op"]]
            deps = [d for d in deps if d != gate["op"]]
        shape = eng.gemm_shapes.get(f"{key}.nb{k}") if rs is None else None
        if shape is not None and p.tile_n == 0:
            # measured at start-up (ops/autotune.py)
            p.tile_m, p.tile_n, p.cta_group = shape["tile_m"], shape["tile_n"], shape["cta_group"]
            p.split_k, p.stream_k = shape["split_k"], shape["stream_k"]
            if gate is not None:
                p.split_k, p.stream_k = 1, 2      # whole tiles in row order (the launcher enforces it as well)
        p.num_ctas = budget.get("gemm", 0)
        p.smem_budget_kb = gemm_smem_budget_kb(eng, tp)
        p.status = _ptr(st)
        if bufs.gemm_ws is not None:
            p.workspace = _ptr(bufs.gemm_ws)
            p.workspace_bytes = bufs.gemm_ws.numel() * bufs.gemm_ws.element_size()
        return g.add(name, p, "gemm", deps=deps, dyn=dyn, layer=layer, nano=k, gated=gated)

    def norm(name, x, wt, out, k, deps, layer, resid=None):
        r0 = starts[k]
        p = NormParams(out=_ptr(out, r0), x=_ptr(x, r0), w=_ptr(wt), resid=c_void_p(0), rows=0, cols=hidden,
                       eps=model.rms_norm_eps)
        return g.add(name, p, S("other"), deps=deps, dyn=[("rows", nb_T[k])], layer=layer, nano=k)

    def attn_front(l, k, lw, pool):
        """norm -> QKV -> RoPE/append -> attention for nano-batch k of layer l."""
        xin = bufs.x[cur]
        gate = None
        if h_normed[k] is not None:
            n1 = h_normed[k]          # the previous all-reduce already wrote the normed rows into h
            h_normed[k] = None
            gate, h_gate[k] = h_gate[k], None
        else:
            n1 = norm(f"L{l}.nb{k}.ln_attn", xin, lw.ln_attn, bufs.h, k, [last_x_writer[k]], l)
        q = gemm(f"L{l}.nb{k}.qkv", bufs.h, lw.wqkv, bufs.qkv, k, bias=lw.bqkv, deps=[n1], layer=l, tile_key="qkv",
                 gate=gate)
        r0 = starts[k]
        rp = RopeAppendParams()
        rp.qkv, rp.ld_qkv = _ptr(bufs.qkv, r0), bufs.qkv.stride(0)
        rp.k_off, rp.v_off, rp.q_off = 0, model.kv_size_local, 2 * model.kv_size_local
        rp.q_out, rp.kv_pool, rp.inv_freq = _ptr(bufs.q_rot, r0), _ptr(pool), _ptr(bufs.inv_freq)
        rp.positions = c_void_p(m["positions"].data_ptr() + 4 * r0)
        rp.token_req = c_void_p(m["token_req"].data_ptr() + 4 * r0)
        rp.kv_indptr, rp.kv_indices = _ptr(m["kv_indptr"]), _ptr(m["kv_indices"])
        rp.T, rp.q_heads, rp.kv_heads, rp.head_dim = 0, model.q_heads_local, model.kv_heads_local, hd
        rp.page_size, rp.num_pages, rp.status = eng.page_size, pool.shape[0], _ptr(st)
        if bufs.rope_table is not None:
            rp.cos_sin = _ptr(bufs.rope_table, r0)   # rows of this nano-batch
        ro = g.add(f"L{l}.nb{k}.rope_append", rp, "gemm" if overlap else S("other"), deps=[q],
                   dyn=[("T", nb_T[k])], layer=l, nano=k)

        def attn_params():
            ap = AttnParams()
            ap.q, ap.out, ap.kv_pool = _ptr(bufs.q_rot), _ptr(bufs.attn_out), _ptr(pool)
            ap.qo_indptr, ap.kv_indptr = _ptr(m["qo_indptr"]), _ptr(m["kv_indptr"])
            ap.kv_indices, ap.kv_last_page_len = _ptr(m["kv_indices"]), _ptr(m["kv_last_page_len"])
            ap.q_heads, ap.kv_heads, ap.head_dim = model.q_heads_local, model.kv_heads_local, hd
            ap.page_size, ap.num_pages, ap.sm_scale = eng.page_size, pool.shape[0], hd ** -0.5
            ap.status = _ptr(st)
            return ap

        # A prompt chunk that straddles the previous nano-batch reads keys that nano-batch appended.
        straddle = [rope_of[(l, k - 1)]] if k > 0 else []
        dp = attn_params()
        dp.num_ctas = budget.get("attn_decode", 0)
        dp.decode_stages = eng.decode_stages
        if tp > 1 and overlap and eng.attn_overlap:
            if dp.num_ctas == 0:
                dp.num_ctas = _ops.sm_count(st.device)   # one CTA per SM: a second would not fit beside a GEMM CTA
            if dp.decode_stages == 0:
                dp.decode_stages = 2 # 64 KB: leaves room for a collective's CTA beside GEMM + decode
        dp.workspace = _ptr(bufs.decode_ws)
        dec_kernel = "nfk_attn_decode_tma" if (eng.decode_impl == "tma" and hd == 128) else "nfk_attn_decode"
        dec = g.add(f"L{l}.nb{k}.attn_decode", dp, S("attn"), deps=[ro], kernel=dec_kernel,
                    dyn=[("req_begin", nb_dec0[k]), ("req_count", nb_decn[k]), ("chunk_pages", chunk_pages),
                         ("max_chunks", max_chunks)], layer=l, nano=k)
        pp = attn_params()
        pp.num_ctas = budget.get("attn_prefill", 0)
        pp.items = _ptr(bufs.nano_items[k])
        # head_dim 128: the tcgen05 kernel; other head sizes: the warp-level mma.sync kernel
        impl = eng.prefill_impl or ("ws" if (hd == 128 and eng.prefill_tc) else "mma")
        if hd != 128:
            impl = "mma"
        pre_kernel = {"ws": "nfk_attn_prefill_ws", "tc": "nfk_attn_prefill_tc", "mma": "nfk_attn_prefill"}[impl]
        pre = g.add(f"L{l}.nb{k}.attn_prefill", pp, prefill_stream, deps=[ro] + straddle, kernel=pre_kernel,
                    dyn=[("num_items", nb_items[k])], layer=l, nano=k)
        rope_of[(l, k)] = ro
        return dec, pre

    comm_ctas = budget.get("comm", 0)
    if overlap and tp > 1 and comm_ctas == 0:
        comm_ctas = default_comm_ctas(tp, bool(getattr(coll, "use_multimem", False)))

    # Residual stream under tensor parallelism: x is a local buffer in which a rank keeps only the
    # rows it owns (row i belongs to rank i % tp) up to date; the K-split GEMMs write their partial
    # products into the symmetric buffer `part`; the collective pulls a row's partials from all
    # ranks, adds the owner's residual row, stores the new residual row locally and pushes only the
    # RMS-normed row to every rank (the next GEMM's input). After the last layer the sums are pushed
    # to every rank instead, so `part` then holds the full final hidden state for sampling.
    x_res = bufs.x[0]
    part = bufs.x[1]
    # Fused GEMM -> reduce-scatter: the K-split GEMMs push their partial rows straight into the owners'
    # slabs from the epilogue (NVLink stores issued tile by tile while later tiles are still in the
    # tensor cores); the collective that follows then only reads local memory and pushes normed rows.
    fuse_rs = tp > 1 and eng.fuse_gemm_rs and hasattr(coll, "rs_slot")
    rs_geom = []
    if fuse_rs:
        row0 = 0
        for k in range(nn):
            cap = (sizes[k] + tp - 1) // tp
            rs_geom.append((row0, cap))
            row0 += cap * tp
        if row0 > part.shape[0]:
            raise ValueError("partial-product buffer too small for the reduce-scatter slabs")

    # nano-batches whose O projection takes the all-gather form
    o1_nanos = set(k for k in eng.o_allgather_nanos if 0 <= k < nn) if tp > 1 else set()
    if o1_nanos:
        if bufs.attn_full is None or any(lw_.wo1 is None for lw_ in w.layers):
            raise ValueError("o_allgather_nanos needs the N-split O weights (wo1) and the attn_full buffer")
        if hidden % (8 * tp) != 0:
            raise ValueError("o_allgather_nanos: hidden size must split into whole 16-byte vectors per rank")

    def rs_slot(k):
        # the slab region of a nano-batch is reused by every fused GEMM of that nano-batch (they are
        # ordered by their collectives' exit handshakes); the flag block is private to each GEMM +
        # collective pair, because flags carry only the iteration's epoch
        return coll.rs_slot(part, *rs_geom[k])

    def o_proj(l, k, lw, dec, pre):
        """O projection -> reduce (+ residual, + fused FFN norm). Returns the op the FFN waits for."""
        if tp == 1:
            if not eng.fuse_gemm_norm:
                o = gemm(f"L{l}.nb{k}.o", bufs.attn_out, lw.wo, x_res, k, residual=x_res, beta=1.0, deps=[dec, pre],
                         layer=l, tile_key="o")
                return norm(f"L{l}.nb{k}.ln_ffn", x_res, lw.ln_ffn, bufs.h, k, [o], l)
            # the FFN's input norm comes out of the same call (fused into the split-K reduce when K is split)
            return gemm(f"L{l}.nb{k}.o", bufs.attn_out, lw.wo, x_res, k, residual=x_res, beta=1.0, deps=[dec, pre],
                        layer=l, tile_key="o", norm=(lw.ln_ffn, bufs.h))
        if k in o1_nanos:
            # All-gather form (the reference's first O-projection scheme, pipeline/src/pipeline.cu:671-682:
            # AG1_GEMV -> O1 -> AG_O1): the ranks' attention outputs are gathered column-wise, the N-split
            # weight gives every rank complete sums for its hidden / tp columns of all rows, and the row owners
            # gather those column blocks (one load per vector instead of one per rank), add the residual,
            # norm and push as after the K-split form. Same bytes on the links as the all-reduce, moved in two
            # steps of which the first is done by the copy engines.
            hs = hidden // tp
            ag = coll.all_gather_columns(g, f"L{l}.nb{k}.ag_attn", bufs.attn_out, bufs.attn_full, starts[k],
                                         nb_T[k], [dec, pre], l, k, stream=net_of(k), status=st)
            o = gemm(f"L{l}.nb{k}.o1", bufs.attn_full, lw.wo1, part[:, w.rank * hs:(w.rank + 1) * hs], k,
                     deps=[ag, last_x_writer[k]], layer=l, tile_key="o1")
            ar1, _ = coll.all_reduce(g, f"L{l}.nb{k}.ag_o", part, starts[k], nb_T[k], hidden, [o], l, k,
                                     stream=net_of(k), norm_w=lw.ln_ffn, norm_out=bufs.h, eps=model.rms_norm_eps,
                                     status=st, num_ctas=comm_ctas, resid=x_res, sum_out=x_res, push_sum=False,
                                     gather_cols=True, **gate_kw(k))
            ffn_gate[k] = take_gate(ar1)
            return ar1
        slab = rs_slot(k) if fuse_rs else None
        o = gemm(f"L{l}.nb{k}.o", bufs.attn_out, lw.wo, None if fuse_rs else part, k,
                 deps=[dec, pre, last_x_writer[k]], layer=l, tile_key="o", rs=slab)
        ar1, _ = coll.all_reduce(g, f"L{l}.nb{k}.ar_o", part, starts[k], nb_T[k], hidden, [o], l, k,
                                 stream=net_of(k), norm_w=lw.ln_ffn, norm_out=bufs.h, eps=model.rms_norm_eps,
                                 status=st, num_ctas=comm_ctas, resid=x_res, sum_out=x_res, push_sum=False,
                                 slab=slab, **gate_kw(k))
        ffn_gate[k] = take_gate(ar1)
        return ar1

    def ffn(l, k, lw, n2):
        """gate/up SwiGLU -> down -> reduce (+ residual, + fused next-layer attention norm)."""
        ffn_down(l, k, lw, ffn_gate_up(l, k, lw, n2))

    def ffn_gate_up(l, k, lw, n2):
        gate, ffn_gate[k] = ffn_gate[k], None
        return gemm(f"L{l}.nb{k}.gate_up", bufs.h, lw.wg, bufs.act, k, swiglu_up=lw.wu, deps=[n2], layer=l,
                    tile_key="gate_up", gate=gate)

    def ffn_down(l, k, lw, gu):
        if tp == 1:
            # the next layer's attention norm comes out of the same call (not after the last layer:
            # the final norm runs on the sampled rows only)
            nxt1 = None if (l + 1 >= model.run_layers or not eng.fuse_gemm_norm) else \
                (w.layers[(l + 1) % model.num_layers].ln_attn, bufs.h)
            d = gemm(f"L{l}.nb{k}.down", bufs.act, lw.wd, x_res, k, residual=x_res, beta=1.0, deps=[gu], layer=l,
                     tile_key="down", norm=nxt1)
            last_x_writer[k] = d
            h_normed[k] = d if nxt1 is not None else None
            return
        last = l + 1 >= model.run_layers
        # the last layer's sum must reach every rank in full (sampling reads arbitrary rows), which
        # the slab form cannot do: it keeps the pull form with push_sum
        slab = rs_slot(k) if (fuse_rs and not last) else None
        d = gemm(f"L{l}.nb{k}.down", bufs.act, lw.wd, None if slab else part, k, deps=[gu], layer=l,
                 tile_key="down", rs=slab)
        nxt = None if last else w.layers[(l + 1) % model.num_layers].ln_attn
        ar2, fused2 = coll.all_reduce(g, f"L{l}.nb{k}.ar_d", part, starts[k], nb_T[k], hidden, [d], l, k,
                                      stream=net_of(k), norm_w=nxt, norm_out=None if last else bufs.h,
                                      eps=model.rms_norm_eps, status=st, num_ctas=comm_ctas, resid=x_res,
                                      sum_out=x_res, push_sum=last, slab=slab, **({} if last else gate_kw(k)))
        last_x_writer[k] = ar2
        h_normed[k] = ar2 if fused2 else None
        h_gate[k] = take_gate(ar2) if fused2 else None

    def offload_layer(l, pool, pace_dep):
        """Layer-by-layer KV offload of retired requests: gather their pages of layer l into a
        staging buffer and copy them to pinned host memory, all on the copy stream beside the
        layer's compute (the reference's PageAggregator + D2H on stream_cpy, pipeline/src/pipeline.cu:701-716)."""
        page_bytes = pool[0].numel() * pool.element_size()
        kp = KvMoveParams(pool=_ptr(pool), staging=_ptr(io.offload_staging), page_ids=_ptr(io.offload_pages),
                          n_pages=0, page_bytes=page_bytes, num_pages=pool.shape[0], direction=0,
                          num_ctas=budget.get("offload", 8) or 8, status=_ptr(st))
        ga = g.add(f"L{l}.kv_gather", kp, "copy" if overlap else "gemm", deps=[pace_dep],
                   dyn=[("n_pages", g.symbol("offload_n"))], layer=l)
        cp = MemcpyParams(dst=c_void_p(0), src=_ptr(io.offload_staging), elem_bytes=page_bytes, count=0)
        g.add(f"L{l}.kv_d2h", cp, "copy" if overlap else "gemm", deps=[ga],
              dyn=[("dst", g.symbol(f"offload_dst_{l}")), ("count", g.symbol("offload_n"))], layer=l)

    rope_of: Dict = {}
    h_normed: List[Optional[int]] = [None] * nn     # op that already wrote normed rows of nano-batch k into h
    # gate_gemm: the GEMM that reads the normed rows starts together with the all-reduce that delivers them
    # and waits per 128-row block (flags raised by the collective as it pushes): all-gather -> GEMM in one
    # pipeline instead of two kernels in sequence
    use_gate = tp > 1 and eng.gate_gemm and hasattr(coll, "last_gate") and not fuse_rs
    h_gate: List[Optional[dict]] = [None] * nn      # gate of the rows in h that the next QKV GEMM reads
    ffn_gate: List[Optional[dict]] = [None] * nn    # ... that the next gate/up GEMM reads

    def gate_kw(k):
        return {"gate_rows_cap": sizes[k]} if use_gate else {}

    def take_gate(op_idx):
        gt = getattr(coll, "last_gate", None) if use_gate else None
        return dict(gt, op=op_idx) if (gt is not None and op_idx is not None) else None
    for l in range(model.run_layers):
        lw = w.layers[l % model.num_layers]
        pool = bufs.kv_pool[l]
        if eng.offload and io is not None and io.offload_staging is not None:
            offload_layer(l, pool, len(g.ops) - 1)
        if overlap and nn > 1 and eng.cross_layer_pipeline and tp > 1:
            # Skewed schedule under tensor parallelism: behind the O projection of nano-batch k the compute
            # stream gets the front-end (QKV, RoPE / append) of the nano-batch whose O projection comes
            # next (k+1 of this layer, or nano-batch 0 of the next layer), then k's FFN. With
            # attn_overlap the decode attention of that next nano-batch then runs on its own stream under
            # k's gate/up and down GEMMs, the all-reduce of k's O output hides under the front-end GEMM,
            # and the one after k's down projection under the next O projection.
            if nn == 2:
                # Two nano-batches A, B, with B one phase behind A. Per period p the compute stream gets
                #   o(B,p-1)  F(A,p)  gate_up(B,p-1)  o(A,p)  down(B,p-1)  gate_up(A,p)  F(B,p)  down(A,p)
                # (F = QKV + RoPE / append). Every op that has to wait for something off the compute stream
                # has a GEMM of the other nano-batch issued in between: decode attention of A under B's
                # gate/up, the all-reduce of A's O output under B's down projection, the all-reduce after
                # A's down projection under B's O projection, and the same for B a phase later. Of all
                # interleavings of the two chains this one leaves the compute stream idle the least when
                # replayed with measured op durations.
                def lw_of(layer):
                    return w.layers[layer % model.num_layers]

                if l == 0:
                    sw_state = {}
                else:
                    sw_state["n2B"] = o_proj(l - 1, 1, lw_of(l - 1), *sw_state.pop("frontB"))
                sw_state["frontA"] = attn_front(l, 0, lw, pool)
                if l > 0:
                    sw_state["guB"] = ffn_gate_up(l - 1, 1, lw_of(l - 1), sw_state.pop("n2B"))
                n2a = o_proj(l, 0, lw, *sw_state.pop("frontA"))
                if l > 0:
                    ffn_down(l - 1, 1, lw_of(l - 1), sw_state.pop("guB"))
                gua = ffn_gate_up(l, 0, lw, n2a)
                sw_state["frontB"] = attn_front(l, 1, lw, pool)
                ffn_down(l, 0, lw, gua)
                if l + 1 == model.run_layers:
                    ffn(l, 1, lw, o_proj(l, 1, lw, *sw_state.pop("frontB")))
                continue
            if l == 0:
                sw_fronts = {0: attn_front(0, 0, lw, pool)}
            for k in range(nn):
                n2 = o_proj(l, k, lw, *sw_fronts.pop(k))
                if k + 1 < nn:
                    sw_fronts[k + 1] = attn_front(l, k + 1, lw, pool)
                elif l + 1 < model.run_layers:
                    sw_fronts[0] = attn_front(l + 1, 0, w.layers[(l + 1) % model.num_layers], bufs.kv_pool[l + 1])
                ffn(l, k, lw, n2)
        elif overlap and nn > 1 and eng.cross_layer_pipeline:
            # Software pipeline across layers (the reference's one-GPU schedule,
            # pipeline/src/pipeline_local.cu:353-431): per nano-batch the compute stream gets
            # O / FFN of layer l followed at once by QKV / RoPE of layer l+1, so the attention of that
            # nano-batch for layer l+1 (attention stream) runs under the O / FFN / QKV GEMMs of the other
            # nano-batches, and is done when its own O projection comes round again.
            if l == 0:
                sw_fronts = [attn_front(0, k, lw, pool) for k in range(nn)]
            nxt_l = l + 1
            for k in range(nn):
                ffn(l, k, lw, o_proj(l, k, lw, *sw_fronts[k]))
                if nxt_l < model.run_layers:
                    sw_fronts[k] = attn_front(nxt_l, k, w.layers[nxt_l % model.num_layers], bufs.kv_pool[nxt_l])
        elif overlap and nn > 1:
            # Issue order per layer: (front_k, o_k) for every nano-batch, then ffn_k for every
            # nano-batch. The all-reduce after o_k then runs (on the net stream, its CTAs sharing SMs
            # with the GEMM CTAs) beside the attention front-end of nano-batch k+1, the one after
            # ffn_k beside ffn_{k+1} or the next layer's front-end: no GEMM waits on a collective
            # that started right before it.
            n2s = []
            if tp > 1 and eng.attn_overlap:
                fronts = [attn_front(l, k, lw, pool) for k in range(nn)]
                for k in range(nn):
                    n2s.append(o_proj(l, k, lw, *fronts[k]))
            else:
                for k in range(nn):
                    dec, pre = attn_front(l, k, lw, pool)
                    n2s.append(o_proj(l, k, lw, dec, pre))
            for k in range(nn):
                ffn(l, k, lw, n2s[k])
        else:
            for k in range(nn):
                dec, pre = attn_front(l, k, lw, pool)
                ffn(l, k, lw, o_proj(l, k, lw, dec, pre))

    # ---- epilogue: sample --------------------------------------------------------------------------
    final_x = bufs.x[0] if tp == 1 else bufs.x[1]
    gp = GatherParams(out=_ptr(bufs.sample_h), inp=_ptr(final_x), rows_idx=_ptr(m["sample_rows"]), n=0,
                      cols=hidden, ld_in=final_x.stride(0), in_rows=final_x.shape[0], status=_ptr(st))
    ga = g.add("gather_last", gp, S("other"), deps=[d for d in last_x_writer if d is not None],
               dyn=[("n", n_sample)])
    fp = NormParams(out=_ptr(bufs.sample_hn), x=_ptr(bufs.sample_h), w=_ptr(w.norm), resid=c_void_p(0), rows=0,
                    cols=hidden, eps=model.rms_norm_eps)
    fn = g.add("final_norm", fp, S("other"), deps=[ga], dyn=[("rows", n_sample)])
    lp = GemmParams()
    lp.A, lp.B, lp.D = _ptr(bufs.sample_hn), _ptr(w.lm_head), _ptr(bufs.logits)
    lp.B2, lp.C, lp.bias = c_void_p(0), c_void_p(0), c_void_p(0)
    lp.lda, lp.ldb, lp.ldd, lp.ldc = bufs.sample_hn.stride(0), w.lm_head.stride(0), bufs.logits.stride(0), 0
    lp.beta, lp.M, lp.N, lp.K = 0.0, 0, w.lm_head.shape[0], hidden
    lp.epilogue, lp.tile_n, lp.num_ctas, lp.status = 0, eng.gemm_tile_n.get("lm_head", 0), 0, _ptr(st)
    if bufs.gemm_ws is not None:
        lp.workspace = _ptr(bufs.gemm_ws)
        lp.workspace_bytes = bufs.gemm_ws.numel() * bufs.gemm_ws.element_size()
    lm = g.add("lm_head", lp, "gemm", deps=[fn], dyn=[("M", n_sample)])
    vl = w.lm_head.shape[0]
    valid = max(0, min(vl, model.vocab_size - w.rank * vl))
    Bcap = bufs.sampled.shape[0]
    if tp == 1:
        ap = ArgmaxParams(idx_out=_ptr(bufs.sampled), val_out=c_void_p(0), logits=_ptr(bufs.logits), rows=0,
                          cols=valid, ld=bufs.logits.stride(0), col_offset=0)
        last = g.add("argmax", ap, S("other") if overlap else "gemm", deps=[lm], dyn=[("rows", n_sample)])
    else:
        ap = ArgmaxParams(idx_out=_ptr(bufs.cand_idx, w.rank), val_out=_ptr(bufs.cand_val, w.rank),
                          logits=_ptr(bufs.logits), rows=0, cols=valid, ld=bufs.logits.stride(0),
                          col_offset=w.rank * vl)
        am = g.add("argmax_local", ap, S("other") if overlap else "gemm", deps=[lm], dyn=[("rows", n_sample)])
        agc = coll.all_gather_candidates(g, bufs, n_sample, [am])
        cp = ArgmaxCombineParams(idx_out=_ptr(bufs.sampled), cand_val=_ptr(bufs.cand_val),
                                 cand_idx=_ptr(bufs.cand_idx), shards=tp, rows=Bcap)
        last = g.add("argmax_combine", cp, S("net"), deps=[agc if agc is not None else am])
    if io is not None:
        c3 = MemcpyParams(dst=c_void_p(0), src=_ptr(bufs.sampled), elem_bytes=4, count=0)
        td = g.add("tokens_d2h", c3, g.ops[last].stream, deps=[last],
                   dyn=[("dst", g.symbol("tokens_dst")), ("count", n_sample)])
        # the status word travels with the tokens, so the host sees a timeout or a bad index in the
        # iteration that had it, not at the end of serving
        c4 = MemcpyParams(dst=c_void_p(0), src=_ptr(st), elem_bytes=4, count=1)
        g.add("status_d2h", c4, g.ops[last].stream, deps=[td], dyn=[("dst", g.symbol("status_dst"))])
    return g
