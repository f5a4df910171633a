"""Per-GPU engine: owns the weights, the paged KV pool, the static activation buffers, the
per-iteration metadata block and the op graph; runs iterations asynchronously.

API (names follow the reference's ``pllm_python`` surface, pipeline/src/pybind.cu:189-283, and its
worker loop, pipeline/src/computeBound.cu:115-193):

``update(plan)``        stage the batch metadata of the next iteration in pinned host memory
``run_async()``         H2D the metadata, launch the whole iteration, D2H the sampled tokens; returns
                        immediately
``run_async_wait()``    block until the oldest launched iteration is done; returns its sampled tokens
``run(plan)``           the three above in sequence
``getPipelineOutput()`` tokens of the last waited iteration

Input token ids of decode requests never visit the host: the embedding op reads them from the
previous iteration's ``sampled`` array on the device through ``feedback_src`` indices
(computeBound.cu:122-150 does this merge on the host in the reference).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..config import EngineConfig, ModelConfig, NanoflowConfig
from ..models.llama import RankWeights
from ..ops import reference as ref
from ..serving.scheduler import BatchPlan
from .graph import OpGraph, PyExecutor
from .pipeline import Buffers, CollectiveHooks, IoSpec, build_graph, gemm_smem_budget_kb

RING = 3                       # host staging slots (iterations in flight + one being formed)
DECODE_MAX_CHUNKS = 16
OFFLOAD_HOST_BYTES = 256 << 20 # pinned host staging per ring slot for the KV offload
GEMM_WS_BYTES = 160 << 20      # fp32 partial sums of split-K / stream-K-tail GEMMs (the GEMMs of one engine share a stream)
DECODE_SPLIT_ROWS = 8192       # workspace rows (request x q head) reserved for split-KV decode


class MetaLayout:
    """Offsets (int32 words) of every per-iteration array inside one contiguous metadata block."""

    def __init__(self, T: int, B: int, nano_sizes: List[int], num_pages: int, offload_cap: int = 0):
        self.T, self.B = T, B
        off = 0
        self.off: Dict[str, int] = {}
        self.size: Dict[str, int] = {}

        def put(name, n):
            nonlocal off
            self.off[name], self.size[name] = off, n
            off += (n + 3) // 4 * 4        # keep every array 16-byte aligned

        for name in ("host_ids", "feedback_src", "positions", "token_req"):
            put(name, T)
        put("qo_indptr", B + 1)
        put("kv_indptr", B + 1)
        put("kv_last_page_len", B)
        put("sample_rows", B)
        self.item_caps = [s + 2 for s in nano_sizes]
        for k, cap in enumerate(self.item_caps):
            put(f"items{k}", cap * 3)
        put("offload_pages", offload_cap)
        self.fixed_words = off
        put("kv_indices", num_pages + B)
        self.total_words = off


class Engine:
    def __init__(self, cfg: NanoflowConfig, weights: RankWeights, *, device: Optional[torch.device] = None,
                 collectives: Optional[CollectiveHooks] = None, num_pages: Optional[int] = None,
                 executor: str = "auto"):
        if not torch.cuda.is_available():
            raise RuntimeError("Engine needs a CUDA device (use runtime.cpu_backend.CpuEngine on CPU)")
        ops.lib()   # fail loudly if the kernel library is missing
        self.cfg, self.model, self.eng = cfg, cfg.model, cfg.engine
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.w = weights
        self.coll = collectives or CollectiveHooks()
        m, e = self.model, self.eng
        if e.page_size != 16:
            raise ValueError("the attention kernels are built for 16-token pages")
        T, B = e.global_batch_size, e.max_batch_size
        self.nano_sizes = e.resolved_nanobatches()
        dev, bf = self.device, torch.bfloat16

        def alloc(*shape, dtype=bf):
            return self.coll.alloc(shape, dtype) if hasattr(self.coll, "alloc") else \
                torch.zeros(*shape, dtype=dtype, device=dev)

        # debug_guards: every local activation buffer sits between guard words that check_status()
        # compares after the iteration (utils/guards.py)
        self.guards = None
        if e.debug_guards:
            from ..utils.guards import GuardedArena
            self.guards = GuardedArena(dev)

        def plain(*shape, dtype=bf, name="activation"):
            if self.guards is not None:
                return self.guards.zeros(name, shape, dtype)
            return torch.zeros(*shape, dtype=dtype, device=dev)

        # x[0]: residual stream (local). x[1]: under TP the symmetric buffer the K-split GEMMs write
        # their partial products into (peers pull from it); on one GPU it aliases x[0].
        x0 = plain(T, m.hidden_size, name="x")
        x = [x0, alloc(T + 8 * len(self.nano_sizes), m.hidden_size) if weights.tp > 1 else x0]
        self.num_pages = int(num_pages or e.num_pages or self._derive_num_pages(T, B))
        # KV offload: pages of requests retired in an iteration are gathered layer by layer and
        # copied to pinned host memory; at most offload_cap pages per iteration.
        self.page_bytes_layer = 2 * m.kv_heads_local * e.page_size * m.head_dim * 2
        self.offload_cap = 0
        if e.offload:
            self.offload_cap = max(16, min(2048, OFFLOAD_HOST_BYTES // (m.run_layers * self.page_bytes_layer)))
        layout = MetaLayout(T, B, self.nano_sizes, self.num_pages, self.offload_cap)
        self.layout = layout
        self.meta_dev = torch.zeros(layout.total_words, dtype=torch.int32, device=dev)
        self.meta_host = [torch.zeros(layout.total_words, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self.meta_np = [t.numpy() for t in self.meta_host]
        view = lambda name: self.meta_dev[layout.off[name]:layout.off[name] + layout.size[name]]
        meta = {n: view(n) for n in ("host_ids", "feedback_src", "positions", "token_req", "qo_indptr",
                                     "kv_indptr", "kv_last_page_len", "sample_rows", "kv_indices")}
        nano_items = [view(f"items{k}").view(-1, 3) for k in range(len(self.nano_sizes))]
        kv_pool = [torch.zeros(self.num_pages, 2, m.kv_heads_local, e.page_size, m.head_dim, dtype=bf, device=dev)
                   for _ in range(m.run_layers)]
        self.bufs = Buffers(
            x=x, h=alloc(T, m.hidden_size) if weights.tp > 1 else plain(T, m.hidden_size, name="h"),
            qkv=plain(T, m.qkv_size_local, name="qkv"), q_rot=plain(T, m.q_size_local, name="q_rot"),
            attn_out=plain(T, m.q_size_local, name="attn_out"), act=plain(T, m.ffn_local, name="act"),
            sample_h=plain(B, m.hidden_size, name="sample_h"), sample_hn=plain(B, m.hidden_size, name="sample_hn"),
            logits=plain(B, weights.lm_head.shape[0], name="logits"),
            cand_val=alloc(weights.tp, B, dtype=torch.float32), cand_idx=alloc(weights.tp, B, dtype=torch.int32),
            sampled=plain(B, dtype=torch.int32, name="sampled"), kv_pool=kv_pool,
            inv_freq=ref.rope_inv_freq(m.head_dim, m.rope_theta, m.rope_scaling).to(dev),
            status=torch.zeros(1, dtype=torch.int32, device=dev),
            decode_ws=torch.empty(DECODE_SPLIT_ROWS * DECODE_MAX_CHUNKS * (m.head_dim + 2), dtype=torch.float32,
                                  device=dev),
            meta=meta, nano_items=nano_items,
            gemm_ws=torch.zeros(GEMM_WS_BYTES // 4, dtype=torch.float32, device=dev),
            rope_table=torch.zeros(T, m.head_dim // 2, 2, dtype=torch.float32, device=dev),
            attn_full=alloc(T, m.q_size_local * weights.tp) if (weights.tp > 1 and e.o_allgather_nanos) else None)
        io = IoSpec(self.meta_dev, layout.fixed_words, layout.off["kv_indices"])
        self.offload_host = None
        if self.offload_cap:
            io.offload_staging = torch.zeros(self.offload_cap, self.page_bytes_layer // 2, dtype=bf, device=dev)
            io.offload_pages = view("offload_pages")
            self.offload_host = [torch.zeros(m.run_layers, self.offload_cap, self.page_bytes_layer // 2,
                                             dtype=bf).pin_memory() for _ in range(RING)]
        self.gemm_tuning: Dict[str, dict] = {}
        if e.autotune_gemm:
            self._autotune_gemms()
        self.graph: OpGraph = build_graph(m, e, weights, self.bufs, self.coll, io)
        self.tokens_host = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self.tokens_np = [t.numpy() for t in self.tokens_host]
        self.status_host = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self.status_np = [t.numpy() for t in self.status_host]
        self.stream = torch.cuda.Stream(device=dev)
        self.done_events = [torch.cuda.Event() for _ in range(RING)]
        self._staged: Optional[dict] = None
        self._inflight: List[dict] = []
        self._iter = 0
        self._last_tokens = np.zeros(0, dtype=np.int32)
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.last_offload = (0, 0)
        self.launches_per_iteration = len(self.graph.ops)
        self.executor_kind = executor
        self._make_executor(executor)

    # ---- GEMM shapes --------------------------------------------------------------------------------
    def _autotune_gemms(self) -> None:
        """Time candidate kernel shapes for the four per-layer GEMMs at every nano-batch size, on this
        engine's buffers and the layers' own weights, and pin the fastest (ops/autotune.py). Shapes
        given in the configuration are kept."""
        from ..ops import autotune
        m, e, w, b = self.model, self.eng, self.w, self.bufs
        budget = e.sm_budget.get("gemm", 0) if e.overlap else 0
        tp1 = w.tp == 1
        x_out = b.x[0] if tp1 else b.x[1]
        L = w.layers
        specs = [("qkv", b.h, [l.wqkv for l in L], None, b.qkv, None, L[0].bqkv),
                 ("o", b.attn_out, [l.wo for l in L], None, x_out, x_out if tp1 else None, None),
                 ("gate_up", b.h, [l.wg for l in L], [l.wu for l in L], b.act, None, None),
                 ("down", b.act, [l.wd for l in L], None, x_out, x_out if tp1 else None, None)]
        o1_nanos = set(e.o_allgather_nanos) if (b.attn_full is not None) else set()
        if o1_nanos:
            hs = m.hidden_size // w.tp
            specs.append(("o1", b.attn_full, [l.wo1 for l in L], None, x_out[:, w.rank * hs:(w.rank + 1) * hs],
                          None, None))
            b.attn_full.normal_()
        for t in (b.h, b.attn_out, b.act):
            t.normal_()
        done: Dict[tuple, dict] = {}
        for k, M in enumerate(self.nano_sizes):
            if M <= 0:
                continue
            for key, a, ws, ups, out, resid, bias in specs:
                name = f"{key}.nb{k}"
                if name in e.gemm_shapes or key in e.gemm_tile_n:
                    continue
                if (key == "o1") != (k in o1_nanos) and key in ("o", "o1"):
                    continue
                if (key, M) not in done:
                    done[(key, M)] = autotune.tune_gemm(
                        a[:M], ws, out[:M], weights_up=ups, residual=None if resid is None else resid[:M],
                        bias=bias, num_ctas=budget, workspace=b.gemm_ws,
                        smem_budget_kb=gemm_smem_budget_kb(e, w.tp))
                r = done[(key, M)]
                e.gemm_shapes[name] = dict(r["best"])
                self.gemm_tuning[name] = dict(M=M, best=r["best"], us=r["us"], auto_us=r["auto_us"])
        torch.cuda.synchronize(self.device)
        for t in (b.h, b.attn_out, b.act, b.qkv, b.x[0], b.x[1], b.attn_full):
            if t is not None:
                t.zero_()

    # ---- sizing -----------------------------------------------------------------------------------
    def _derive_num_pages(self, T: int, B: int) -> int:
        m, e = self.model, self.eng
        free, total = torch.cuda.mem_get_info(self.device)
        act = 2 * T * (3 * m.hidden_size + m.qkv_size_local + 2 * m.q_size_local + m.ffn_local)
        act += 2 * B * (2 * m.hidden_size + self.w.lm_head.shape[0]) + (256 << 20)
        if e.o_allgather_nanos and self.w.tp > 1:
            act += 2 * T * m.q_size_local * self.w.tp
        budget = free - (total * (1.0 - e.gpu_mem_fraction)) - act
        page_bytes = 2 * m.kv_heads_local * e.page_size * m.head_dim * 2 * m.run_layers
        n = int(budget // page_bytes)
        if n < 64:
            raise RuntimeError(f"not enough GPU memory for a KV pool ({free >> 20} MiB free)")
        return n

    def _make_executor(self, kind: str) -> None:
        self.native = None
        single = not (self.eng.overlap or any(op.stream != "gemm" for op in self.graph.ops))
        if kind in ("auto", "native", "graph"):
            try:
                from .native import NativeExecutor
                self.native = NativeExecutor(self.graph, self.stream, single_stream=single,
                                             device=self.device.index or 0,
                                             use_cuda_graph=(kind == "graph" or self.eng.use_cuda_graph))
            except ImportError:
                if kind != "auto":
                    raise
        self.py_exec = None if self.native is not None else PyExecutor(self.graph, single_stream=single)

    # ---- per-iteration ----------------------------------------------------------------------------
    def update(self, plan: BatchPlan) -> None:
        """Write the plan's arrays into the next pinned staging slot and compute the symbol table."""
        lay = self.layout
        if plan.num_tokens > lay.T or plan.num_requests > lay.B:
            raise ValueError("plan exceeds the configured dense batch / request capacity")
        slot = self._iter % RING
        buf = self.meta_np[slot]

        def put(name, arr):
            o = lay.off[name]
            if arr.size > lay.size[name]:
                raise ValueError(f"{name}: {arr.size} entries exceed capacity {lay.size[name]}")
            buf[o:o + arr.size] = arr

        put("host_ids", plan.host_ids); put("feedback_src", plan.feedback_src)
        put("positions", plan.positions); put("token_req", plan.token_req)
        put("qo_indptr", plan.qo_indptr); put("kv_indptr", plan.kv_indptr)
        put("kv_last_page_len", plan.kv_last_page_len); put("sample_rows", plan.sample_rows)
        put("kv_indices", plan.kv_indices)
        sym: Dict[str, int] = {"T": plan.num_tokens, "n_sample": int(plan.sample_rows.size)}
        if len(plan.nano) != len(self.nano_sizes):
            raise ValueError("plan was cut for a different nano-batch configuration")
        for k, nb in enumerate(plan.nano):
            put(f"items{k}", nb.items.reshape(-1))
            sym[f"nb{k}_T"], sym[f"nb{k}_items"] = nb.token_count, int(nb.items.shape[0])
            sym[f"nb{k}_dec_begin"], sym[f"nb{k}_dec_count"] = nb.dec_begin, nb.dec_count
            if f"nb{k}_own_rows" in self.graph.symbols:     # rows of the nano-batch this rank owns (row i: rank i % tp)
                tp_, rk = self.w.tp, getattr(self.coll, "rank", 0)
                sym[f"nb{k}_own_rows"] = max(0, (nb.token_count - rk + tp_ - 1) // tp_)
            if f"nb{k}_wire_us" in self.graph.symbols:       # sleeps standing in for absent ranks (virtual TP)
                sym[f"nb{k}_wire_us"] = int(nb.token_count * getattr(self.coll, "fake_wire_us_per_row", 0.0))
        n_off = 0
        if self.offload_cap:
            pages = plan.retired_pages if plan.retired_pages is not None else np.zeros(0, dtype=np.int32)
            n_off = min(int(pages.size), self.offload_cap)
            put("offload_pages", pages[:n_off])
            sym["offload_n"] = n_off
            host = self.offload_host[slot]
            for l in range(self.model.run_layers):
                sym[f"offload_dst_{l}"] = host.data_ptr() + l * host.stride(0) * host.element_size()
        cp, mc = self._decode_split(plan)
        sym["decode_chunk_pages"], sym["decode_max_chunks"] = cp, mc
        self._staged = dict(slot=slot, sym=sym, n_sample=int(plan.sample_rows.size),
                            kv_words=int(plan.kv_indices.size), plan=plan, n_offload=n_off)

    def _decode_split(self, plan: BatchPlan):
        if self.eng.decode_chunk_pages > 0:
            cp = self.eng.decode_chunk_pages
        else:
            items = plan.num_decode * self.model.kv_heads_local
            target = 2 * ops.sm_count(self.device) * 2      # two rounds of two CTAs per SM
            if items == 0 or items >= target or plan.max_kv_pages <= 16:
                return 0, 1
            want = min(DECODE_MAX_CHUNKS, math.ceil(target / items))
            cp = max(8, math.ceil(plan.max_kv_pages / want))
        mc = max(1, math.ceil(plan.max_kv_pages / cp))
        if mc > DECODE_MAX_CHUNKS or plan.num_decode * self.model.q_heads_local > DECODE_SPLIT_ROWS:
            return 0, 1
        return cp, mc

    def run_async(self, timed: bool = False) -> None:
        st = self._staged
        if st is None:
            raise RuntimeError("run_async without update")
        if len(self._inflight) >= RING - 1:
            raise RuntimeError("too many iterations in flight; call run_async_wait first")
        lay, slot = self.layout, st["slot"]
        sym = st["sym"]
        # The graph starts with the metadata H2D copies (on the iteration's first stream, ordered
        # after the previous iteration) and ends with the D2H copy of the sampled tokens.
        sym["meta_src"] = self.meta_host[slot].data_ptr()
        sym["kv_src"] = self.meta_host[slot].data_ptr() + 4 * lay.off["kv_indices"]
        sym["kv_words"] = st["kv_words"]
        sym["tokens_dst"] = self.tokens_host[slot].data_ptr()
        sym["status_dst"] = self.status_host[slot].data_ptr()
        sym["epoch"] = self._iter + 1      # collective flag epoch: same on every rank, never reset
        if self.native is not None:
            st["ticket"] = self.native.submit(sym, timed)
        else:
            with torch.cuda.stream(self.stream):
                self.py_exec.timing = timed
                self.py_exec.run(sym, main_stream=self.stream)
                self.done_events[slot].record(self.stream)
        self.h2d_bytes_last = 4 * (lay.fixed_words + st["kv_words"])
        self.d2h_bytes_last = 4 * st["n_sample"] + 4 + st.get("n_offload", 0) * self.page_bytes_layer * self.model.run_layers
        self._inflight.append(st)
        self._staged = None
        self._iter += 1

    def run_async_wait(self) -> np.ndarray:
        if not self._inflight:
            raise RuntimeError("nothing in flight")
        st = self._inflight.pop(0)
        if self.native is not None:
            self.native.wait(st["ticket"])
        else:
            self.done_events[st["slot"]].synchronize()
        self._last_tokens = self.tokens_np[st["slot"]][:st["n_sample"]].copy()
        self.last_offload = (st["slot"], st.get("n_offload", 0))
        code = int(self.status_np[st["slot"]][0]) & 0xFFFFFFFF
        if code:
            # a bounded wait ran out (peer gone) or an index was out of range in this iteration: its
            # tokens cannot be trusted, so stop here rather than at the end of serving
            self.status_np[st["slot"]][0] = 0
            self.bufs.status.zero_()
            raise RuntimeError(f"engine iteration {self._iter - len(self._inflight) - 1}: device status 0x{code:x} "
                               f"({ops.STATUS_CODES.get(code & 0xF00, '?')})")
        return self._last_tokens

    def offloaded_pages(self) -> Optional[torch.Tensor]:
        """Host copy [layers, n, page_elems] of the pages offloaded by the last waited iteration."""
        if self.offload_host is None:
            return None
        slot, n = self.last_offload
        return self.offload_host[slot][:, :n]

    def timeline(self):
        """(op name, stream class, start_us, end_us) of the last iteration run with ``timed=True``."""
        return self.native.timeline() if self.native is not None else list(self.py_exec.timeline)

    def run(self, plan: BatchPlan) -> np.ndarray:
        self.update(plan)
        self.run_async()
        return self.run_async_wait()

    def getPipelineOutput(self) -> np.ndarray:
        return self._last_tokens

    @property
    def in_flight(self) -> int:
        return len(self._inflight)

    def check_status(self) -> None:
        ops.check_status(self.bufs.status, "engine iteration")
        if self.guards is not None:
            torch.cuda.synchronize(self.device)
            bad = self.guards.check()
            if bad:
                self.guards.restore()
                raise RuntimeError("write outside an activation buffer: " +
                                   ", ".join(f"{n} ({side} guard, byte {off})" for n, side, off in bad))

    def finalize(self) -> None:
        torch.cuda.synchronize(self.device)
        self._inflight.clear()
        if self.native is not None:
            self.native.close()
