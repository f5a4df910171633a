"""Tensor-parallel collective ops for the op graph and for direct use.

:class:`TpCollectives` owns the symmetric heap of this rank, hands out symmetric tensors to the
engine (residual buffers, normed activations, arg-max candidates) and appends all-reduce /
all-gather ops to the graph. Every op instance gets its own 128-byte flag block; the epoch that
the flags carry is the iteration counter symbol ``epoch``, so nothing is ever reset.
"""
from __future__ import annotations

import ctypes
from ctypes import Structure, byref, c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence

import torch

from .. import ops as _ops
from ..runtime.graph import KERNEL_OF, OpGraph
from ..runtime.pipeline import Buffers, CollectiveHooks
from .symm import SymmetricHeap


class CommCtx(Structure):
    _fields_ = [("heap", c_void_p * 8), ("rank", c_int), ("nranks", c_int)]


class AllReduceParams(Structure):
    _fields_ = [("ctx", CommCtx), ("buf_off", c_longlong), ("flag_off", c_longlong), ("rows", c_int),
                ("cols", c_int), ("ld", c_longlong), ("epoch", c_int), ("num_ctas", c_int),
                ("norm_w", c_void_p), ("norm_out_off", c_longlong), ("norm_ld", c_longlong), ("eps", c_float),
                ("status", c_void_p), ("push_sum", c_int), ("resid", c_void_p), ("resid_ld", c_longlong),
                ("sum_out", c_void_p), ("sum_ld", c_longlong), ("src_mode", c_int), ("slab_rows", c_int),
                ("wide", c_int), ("gate_off", c_longlong), ("gate_cnt", c_void_p), ("push_mode", c_int),
                ("mc_heap", c_void_p)]


class AllGatherParams(Structure):
    _fields_ = [("ctx", CommCtx), ("buf_off", c_longlong), ("shard_bytes", c_longlong),
                ("shard_stride", c_longlong), ("flag_off", c_longlong), ("epoch", c_int), ("num_ctas", c_int),
                ("handshake_in", c_int), ("status", c_void_p), ("rows", c_int), ("row_stride", c_longlong)]


class BarrierParams(Structure):
    _fields_ = [("ctx", CommCtx), ("flag_off", c_longlong), ("epoch", c_int), ("status", c_void_p)]


KERNEL_OF[AllReduceParams] = "nfk_allreduce"
KERNEL_OF[AllGatherParams] = "nfk_allgather"
KERNEL_OF[BarrierParams] = "nfk_comm_barrier"

FLAG_BYTES = 128


class TpCollectives(CollectiveHooks):
    def __init__(self, rank: int, world: int, device: torch.device, heap_bytes: int = 1 << 30,
                 num_ctas: int = 0, fuse_norm: bool = True, backend: str = ""):
        if world > 8:
            raise ValueError("at most 8 ranks (one NVSwitch domain)")
        self.rank, self.tp, self.device = rank, world, device
        self.heap = SymmetricHeap(rank, world, device, heap_bytes, backend=backend)
        # all-reduces go through the NVSwitch (multimem) when the heap has a multicast mapping and there are
        # eight ranks: that is where it was timed (168 against 210-228 us alone). With two ranks half of a
        # row's partial sums are local and the peer-load form is as fast; four ranks keep the peer-load form,
        # which is the one that has run there (set use_multimem to try the other).
        self.use_multimem = self.heap.mc_base != 0 and world >= 8
        self.last_gate = None
        self.num_ctas = num_ctas or _ops.sm_count(device)
        self.fuse_norm = fuse_norm
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.fake_wire_us_per_row = 0.0     # see all_reduce(): sleep standing in for absent ranks
        self.wide = False                   # all-reduce with twice the loads in flight per phase (8 ranks)
        self.push_by_copy = False           # normed rows reach the peers by copy-engine copies (see all_reduce)
        self._epoch = 0
        self._adhoc_flags = self.heap.alloc_bytes(FLAG_BYTES)

    @classmethod
    def for_analysis(cls, rank: int, world: int, heap_bytes: int = 64 << 20) -> "TpCollectives":
        """A TpCollectives whose "heap" is a host tensor: builds graphs for static checks (dependency
        checker, op counts) on a machine without GPUs. Its ops must never be launched."""
        self = cls.__new__(cls)
        self.rank, self.tp, self.device = rank, world, torch.device("cpu")
        self.num_ctas, self.fuse_norm = 16, True
        self.use_multimem = False
        self.last_gate = None
        self.push_by_copy = False
        self.fake_wire_us_per_row = 0.0
        self.wide = False
        self.status = torch.zeros(1, dtype=torch.int32)
        self._epoch = 0

        class _HostHeap:
            def __init__(h):
                h.buf = torch.zeros(heap_bytes, dtype=torch.uint8)
                h.base, h.nbytes, h._bump = h.buf.data_ptr(), heap_bytes, 0
                h.peer_base = [h.base] * world

            def alloc_bytes(h, n, align=256):
                off = (h._bump + align - 1) // align * align
                if off + n > h.nbytes:
                    raise RuntimeError("analysis heap exhausted")
                h._bump = off + n
                return off

            def alloc(h, shape, dtype):
                n = 1
                for x in shape:
                    n *= int(x)
                nb = n * torch.empty(0, dtype=dtype).element_size()
                off = h.alloc_bytes(max(nb, 16))
                return h.buf[off:off + nb].view(dtype).view(*shape)

            def offset_of(h, t):
                return t.data_ptr() - h.base

            def close(h):
                pass

        self.heap = _HostHeap()
        self._adhoc_flags = self.heap.alloc_bytes(FLAG_BYTES)
        return self

    # ---- plumbing ---------------------------------------------------------------------------------
    def ctx(self) -> CommCtx:
        c = CommCtx()
        for r in range(self.tp):
            c.heap[r] = self.heap.peer_base[r]
        c.rank, c.nranks = self.rank, self.tp
        return c

    def alloc(self, shape, dtype) -> torch.Tensor:
        return self.heap.alloc(shape, dtype)

    def new_flags(self) -> int:
        return self.heap.alloc_bytes(FLAG_BYTES)

    # ---- graph hooks --------------------------------------------------------------------------------
    def all_reduce(self, g: OpGraph, name: str, buf: torch.Tensor, row0: int, rows_sym: str, cols: int,
                   deps, layer: int, nano: int, stream: str = "net", norm_w: Optional[torch.Tensor] = None,
                   norm_out: Optional[torch.Tensor] = None, eps: float = 1e-5, status=None, num_ctas: int = 0,
                   resid: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None,
                   push_sum: bool = True, slab: Optional[dict] = None, gate_rows_cap: int = 0,
                   gather_cols: bool = False):
        """Append a reduction of ``buf`` rows [row0, row0+rows) over all ranks.

        ``gather_cols``: rank r's ``buf`` holds columns [r*cols/tp, (r+1)*cols/tp) of the rows (an N-split
        GEMM wrote them); the row owners gather the blocks instead of summing (kernel src_mode 2), the rest
        (residual, stored sum, norm, pushes) is the same.

        ``gate_rows_cap`` > 0 (with a fused norm): the op also raises row-block flags as it pushes the
        normed rows; ``self.last_gate`` then holds what the consumer GEMM needs (see GemmParams.gate_flags).

        With ``slab`` (from :meth:`rs_slot`) the partial rows were pushed into local slabs by a GEMM
        with the reduce-scatter epilogue: the op then reads locally and shares the GEMM's flag block.

        ``resid`` / ``sum_out`` are local tensors (rows owned by this rank are read / written);
        ``push_sum`` writes the sum back into ``buf`` on every rank; ``norm_w`` + ``norm_out`` push
        the RMS-normed sum into the symmetric ``norm_out`` on every rank."""
        p = AllReduceParams()
        p.ctx = self.ctx()
        esz = buf.element_size()
        if slab is not None:
            p.buf_off, p.flag_off = slab["slab_off"], slab["flag_off"]
            p.src_mode, p.slab_rows = 1, slab["rows_cap"]
        else:
            p.buf_off = self.heap.offset_of(buf) + row0 * buf.stride(0) * esz
            p.flag_off = self.new_flags()
            if gather_cols:
                p.src_mode = 2
        p.rows, p.cols, p.ld = 0, cols, buf.stride(0)
        p.epoch, p.num_ctas = 0, num_ctas or self.num_ctas
        fused = norm_w is not None and norm_out is not None
        if fused:
            p.norm_w = norm_w.data_ptr()
            p.norm_out_off = self.heap.offset_of(norm_out) + row0 * norm_out.stride(0) * esz
            p.norm_ld, p.eps = norm_out.stride(0), eps
        p.push_sum = 1 if push_sum else 0
        if resid is not None:
            p.resid, p.resid_ld = resid.data_ptr() + row0 * resid.stride(0) * esz, resid.stride(0)
        if sum_out is not None:
            p.sum_out, p.sum_ld = sum_out.data_ptr() + row0 * sum_out.stride(0) * esz, sum_out.stride(0)
        p.status = (status if status is not None else self.status).data_ptr()
        p.wide = 1 if self.wide else 0
        if self.use_multimem and slab is None and not gather_cols:
            p.mc_heap = self.heap.mc_base
        self.last_gate = None
        if gate_rows_cap > 0 and fused and self.fake_wire_us_per_row <= 0:
            blocks = (gate_rows_cap + 127) // 128
            p.gate_off = self.heap.alloc_bytes(blocks * 8 * 4)
            cnt = torch.zeros(blocks, dtype=torch.int32, device=self.device)
            self._gate_keep = getattr(self, "_gate_keep", []) + [cnt]
            p.gate_cnt = cnt.data_ptr()
            self.last_gate = {"flags": self.heap.base + p.gate_off, "nranks": self.tp}
        by_copy = (self.push_by_copy and fused and self.tp > 1 and slab is None and not push_sum
                   and self.last_gate is None and nano >= 0)
        if by_copy:
            p.push_mode = 1
        idx = g.add(name, p, stream, deps=deps, dyn=[("rows", rows_sym), ("epoch", g.symbol("epoch"))],
                    layer=layer, nano=nano)
        if by_copy:
            # The kernel has left this rank's normed rows (rows rank, rank + tp, ...) in its own copy of
            # norm_out. The copy engines deliver them: one strided copy per peer (each row is contiguous, the
            # rows are tp rows apart), behind the kernel on the same stream, so no SM is involved in the
            # half of the collective that moves the most bytes into a GPU; a barrier then tells every rank
            # that its copy of norm_out is complete. The row count is the symbol nb<k>_own_rows.
            from ..runtime.graph import Memcpy2DParams
            row_bytes = norm_out.stride(0) * esz
            first = p.norm_out_off + self.rank * row_bytes
            for step in range(1, self.tp):
                peer = (self.rank + step) % self.tp
                c = Memcpy2DParams()
                c.dst, c.src = self.heap.peer_base[peer] + first, self.heap.base + first
                c.dpitch = c.spitch = self.tp * row_bytes
                c.width, c.height = cols * esz, 0
                idx = g.add(f"{name}.push{peer}", c, stream, deps=[idx],
                            dyn=[("height", g.symbol(f"nb{nano}_own_rows"))], layer=layer, nano=nano)
            b = BarrierParams()
            b.ctx, b.flag_off, b.epoch = self.ctx(), self.new_flags(), 0
            b.status = p.status
            idx = g.add(f"{name}.done", b, stream, deps=[idx], dyn=[("epoch", g.symbol("epoch"))],
                        layer=layer, nano=nano)
        if self.fake_wire_us_per_row > 0 and nano >= 0:
            # Stand-in for the time on the wire when the other ranks are not there (virtual tensor
            # parallelism on one GPU): a one-thread sleep on the collective's stream, as long as the
            # nano-batch's rows times ``fake_wire_us_per_row``. The reference does the same with its
            # SleepWrapper when built without ENABLE_NETWORK (pipeline/include/pipeline.h:98-100).
            from ..runtime.graph import SleepParams
            idx = g.add(name + ".wire", SleepParams(0), stream, deps=[idx],
                        dyn=[("micros", g.symbol(f"nb{nano}_wire_us"))], layer=layer, nano=nano)
        return idx, fused

    def all_gather_columns(self, g: OpGraph, name: str, src: torch.Tensor, dst: torch.Tensor, row0: int,
                           rows_sym: str, deps, layer: int, nano: int, stream: str = "net", status=None):
        """Append a column-wise all-gather done by the copy engines: rows [row0, row0 + rows) of the local
        ``src`` [T, w] become column block ``rank`` of the same rows of the symmetric ``dst`` [T, tp * w] on
        every rank (one strided copy per rank, own copy included), closed by a barrier; no SM moves data. The
        reference gathers the attention output this way in front of its N-split O projection
        (pipeline/src/pipeline.cu:671-677, ``AG1_GEMV``).

        A peer may still be reading its ``dst`` rows from the previous use when this rank's copy arrives
        unless the caller orders them: in the pipelines every use of ``dst`` is followed by a collective with
        an entry handshake that this rank's next attention depends on, which gives that order."""
        from ..runtime.graph import Memcpy2DParams
        esz = src.element_size()
        w_bytes = src.shape[1] * esz
        if dst.shape[1] % src.shape[1] != 0 or dst.shape[1] < self.tp * src.shape[1] or dst.stride(1) != 1 \
                or src.stride(1) != 1:
            raise ValueError("column-wise all-gather: dst must be [rows, tp * w] for src [rows, w]")
        dst_off = self.heap.offset_of(dst) + row0 * dst.stride(0) * esz + self.rank * w_bytes
        idx = None
        for step in range(self.tp):
            peer = (self.rank + step) % self.tp
            c = Memcpy2DParams()
            c.dst, c.src = self.heap.peer_base[peer] + dst_off, src.data_ptr() + row0 * src.stride(0) * esz
            c.dpitch, c.spitch = dst.stride(0) * esz, src.stride(0) * esz
            c.width, c.height = w_bytes, 0
            idx = g.add(f"{name}.copy{peer}", c, stream, deps=list(deps) if idx is None else [idx],
                        dyn=[("height", rows_sym)], layer=layer, nano=nano)
        b = BarrierParams()
        b.ctx, b.flag_off, b.epoch = self.ctx(), self.new_flags(), 0
        b.status = (status if status is not None else self.status).data_ptr()
        return g.add(f"{name}.done", b, stream, deps=[idx], dyn=[("epoch", g.symbol("epoch"))],
                     layer=layer, nano=nano)

    def rs_slot(self, part: torch.Tensor, slab_row0: int, rows_cap: int) -> dict:
        """Slab + flag block for one fused GEMM -> reduce-scatter: ``part`` rows
        [slab_row0, slab_row0 + tp * rows_cap) hold, per source rank, the partial rows this rank owns."""
        return {"slab_off": self.heap.offset_of(part) + slab_row0 * part.stride(0) * part.element_size(),
                "rows_cap": rows_cap, "flag_off": self.new_flags(), "heap": list(self.heap.peer_base),
                "rank": self.rank, "nranks": self.tp}

    def all_gather_candidates(self, g: OpGraph, bufs: Buffers, rows_sym: str, deps):
        """cand_val / cand_idx are [tp, B] symmetric arrays; every rank pushes its row to all peers."""
        last = None
        for t, nm in ((bufs.cand_val, "val"), (bufs.cand_idx, "idx")):
            p = AllGatherParams()
            p.ctx = self.ctx()
            p.buf_off = self.heap.offset_of(t)
            p.shard_stride = t.stride(0) * t.element_size()
            p.shard_bytes = p.shard_stride
            p.flag_off = self.new_flags()
            p.epoch, p.num_ctas, p.handshake_in = 0, 2, 1
            p.status = self.status.data_ptr()
            last = g.add(f"ag_cand_{nm}", p, "net", deps=list(deps) + ([last] if last is not None else []),
                         dyn=[("epoch", g.symbol("epoch"))])
        return last

    # ---- direct (eager) calls, used by tests and micro-benchmarks --------------------------------------
    def _next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    def all_reduce_(self, buf: torch.Tensor, *, norm_w=None, norm_out=None, eps: float = 1e-5,
                    num_ctas: int = 0, flag_off: Optional[int] = None, epoch: Optional[int] = None,
                    rows: Optional[int] = None, resid: Optional[torch.Tensor] = None,
                    sum_out: Optional[torch.Tensor] = None, push_sum: bool = True):
        """In-place sum of a symmetric bf16 [rows, cols] tensor over all ranks (launches on the
        current stream). All ranks must call it the same number of times with the same flag block."""
        p = AllReduceParams()
        p.ctx = self.ctx()
        p.buf_off = self.heap.offset_of(buf)
        p.flag_off = self._adhoc_flags if flag_off is None else flag_off
        p.rows, p.cols, p.ld = (buf.shape[0] if rows is None else rows), buf.shape[1], buf.stride(0)
        p.epoch = self._next_epoch() if epoch is None else epoch
        p.num_ctas = num_ctas or self.num_ctas
        if norm_w is not None:
            p.norm_w = norm_w.data_ptr()
            p.norm_out_off = self.heap.offset_of(norm_out)
            p.norm_ld, p.eps = norm_out.stride(0), eps
        p.push_sum = 1 if push_sum else 0
        if resid is not None:
            p.resid, p.resid_ld = resid.data_ptr(), resid.stride(0)
        if sum_out is not None:
            p.sum_out, p.sum_ld = sum_out.data_ptr(), sum_out.stride(0)
        p.status = self.status.data_ptr()
        p.wide = 1 if self.wide else 0
        if self.use_multimem:
            p.mc_heap = self.heap.mc_base
        rc = _ops.lib().nfk_allreduce(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"nfk_allreduce: {_ops.ERRORS.get(rc, rc)}")
        return buf

    def all_gather_(self, buf: torch.Tensor, *, num_ctas: int = 0):
        """buf is a symmetric [world, ...] tensor whose row ``rank`` holds this rank's shard."""
        p = AllGatherParams()
        p.ctx = self.ctx()
        p.buf_off = self.heap.offset_of(buf)
        p.shard_stride = buf.stride(0) * buf.element_size()
        p.shard_bytes = p.shard_stride
        p.flag_off = self._adhoc_flags
        p.epoch, p.num_ctas, p.handshake_in = self._next_epoch(), num_ctas or self.num_ctas, 1
        p.status = self.status.data_ptr()
        rc = _ops.lib().nfk_allgather(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"nfk_allgather: {_ops.ERRORS.get(rc, rc)}")
        return buf

    def all_gather_columns_(self, buf: torch.Tensor, *, num_ctas: int = 0):
        """Column-wise all-gather: ``buf`` is a symmetric [rows, world * w] tensor whose column block
        ``rank`` this rank has filled; afterwards every rank holds all blocks. The reference gathers the
        attention output and the N-split O projection this way (pipeline/src/comm.cu:116-167,
        ``columnwiseAllgatherKernelEntryPoint``)."""
        rows, width = buf.shape
        if buf.stride(1) != 1 or width % self.tp != 0:
            raise ValueError("column-wise all-gather needs unit column stride and world | columns")
        esz = buf.element_size()
        p = AllGatherParams()
        p.ctx = self.ctx()
        p.buf_off = self.heap.offset_of(buf)
        p.shard_bytes = p.shard_stride = (width // self.tp) * esz
        p.rows, p.row_stride = rows, buf.stride(0) * esz
        if rows == 1:
            p.rows = 0                       # one row is the flat form
        p.flag_off = self._adhoc_flags
        p.epoch, p.num_ctas, p.handshake_in = self._next_epoch(), num_ctas or self.num_ctas, 1
        p.status = self.status.data_ptr()
        rc = _ops.lib().nfk_allgather(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"nfk_allgather: {_ops.ERRORS.get(rc, rc)}")
        return buf

    def reduce_scatter_(self, buf: torch.Tensor, out: torch.Tensor, *, rows: Optional[int] = None,
                        resid: Optional[torch.Tensor] = None, num_ctas: int = 0):
        """Sum of a symmetric bf16 [rows, cols] tensor over all ranks, scattered by rows: rank r gets
        rows r, r + world, r + 2*world, ... written into the same rows of the local tensor ``out``
        (its other rows, and ``buf`` on every rank, are left as they are). The pull phase of the
        all-reduce on its own (pipeline/src/comm.cu:169-282, ``reduceScatterKernel``; the reference
        gives each rank a contiguous block of rows, here ownership is interleaved so that any prefix of
        the rows is spread evenly)."""
        return self.all_reduce_(buf, rows=rows, resid=resid, sum_out=out, push_sum=False, num_ctas=num_ctas)

    # ---- copy-engine forms: peer-to-peer cudaMemcpyAsync, one copy per peer on a stream of its own -----
    def _peer_streams(self):
        if not hasattr(self, "_pstreams"):
            self._pstreams = [torch.cuda.Stream(device=self.device) for _ in range(self.tp)]
        return self._pstreams

    def _copy_to_peer(self, peer: int, dst_off: int, src: torch.Tensor, stream) -> None:
        from ..runtime.graph import MemcpyParams
        p = MemcpyParams(dst=self.heap.peer_base[peer] + dst_off, src=src.data_ptr(), elem_bytes=src.element_size(),
                         count=src.numel())
        rc = _ops.lib().nfk_memcpy_p(byref(p), c_void_p(stream.cuda_stream))
        if rc != 0:
            raise RuntimeError(f"peer copy: {_ops.ERRORS.get(rc, rc)}")

    def _fan_out(self, copies) -> None:
        """Run ``copies`` = [(peer, dst_off, src)] on the per-peer streams between two barriers: peers are
        done with the destination before the first byte lands, and see all of it after the second."""
        cur = torch.cuda.current_stream()
        self.barrier_()
        start = torch.cuda.Event()
        start.record(cur)
        streams = self._peer_streams()
        for peer, dst_off, src in copies:
            st = streams[peer]
            st.wait_event(start)
            self._copy_to_peer(peer, dst_off, src, st)
            done = torch.cuda.Event()
            done.record(st)
            cur.wait_event(done)
        self.barrier_()

    def all_gather_copy_(self, buf: torch.Tensor):
        """All-gather of a symmetric [world, ...] tensor (row ``rank`` filled locally) by the copy engines
        instead of SMs: one peer-to-peer copy per destination, each on its own stream. Counterpart of the
        reference's ``NetAllGatherAsync`` (pipeline/include/netWrapper.cuh:501-559)."""
        if not buf[self.rank].is_contiguous():
            raise ValueError("shards must be contiguous")
        off = self.heap.offset_of(buf) + self.rank * buf.stride(0) * buf.element_size()
        self._fan_out([(r, off, buf[self.rank]) for r in range(self.tp) if r != self.rank])
        return buf

    def reduce_scatter_copy_(self, buf: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor):
        """Reduce-scatter of contiguous shards by the copy engines: ``buf`` [world, n] holds this rank's
        partial sums (any memory), ``scratch`` is a symmetric [world, n] tensor of the same dtype; every
        rank copies its shard ``r`` into row ``rank`` of rank r's ``scratch``, and after the barrier adds up
        the rows it received (fp32 accumulation) into ``out`` [n]. Counterpart of the reference's
        ``NetReduceScatterAsync`` + ``asyncReduceKernel`` (pipeline/include/netWrapper.cuh:562-634,
        pipeline/src/comm.cu:487-530)."""
        if buf.shape != scratch.shape or buf.shape[0] != self.tp or not buf.is_contiguous() or not scratch.is_contiguous():
            raise ValueError("buf and scratch must be contiguous [world, n] tensors")
        row_bytes = scratch.stride(0) * scratch.element_size()
        base = self.heap.offset_of(scratch) + self.rank * row_bytes
        scratch[self.rank].copy_(buf[self.rank])
        self._fan_out([(r, base, buf[r]) for r in range(self.tp) if r != self.rank])
        out.copy_(scratch.float().sum(dim=0).to(out.dtype))      # local memory only
        return out

    def barrier_(self):
        p = BarrierParams()
        p.ctx, p.flag_off, p.epoch = self.ctx(), self._adhoc_flags, self._next_epoch()
        p.status = self.status.data_ptr()
        rc = _ops.lib().nfk_comm_barrier(byref(p), c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"nfk_comm_barrier: {_ops.ERRORS.get(rc, rc)}")

    def check_status(self):
        _ops.check_status(self.status, "collective")

    def close(self):
        self.heap.close()
