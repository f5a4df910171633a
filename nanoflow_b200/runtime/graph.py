"""Declarative per-iteration op graph.

A graph is an ordered list of :class:`Op`: a kernel entry point of ``libnanoflow_kernels.so`` in the
uniform ``int fn(const params*, cudaStream_t)`` form, its parameter block (a ``ctypes.Structure``),
the *stream class* it runs on (``gemm``, ``attn``, ``net``, ``other``, ``copy``, ``attn2``, ``net2``), the ops it must
wait for, and a list of *dynamic fields*: integer members of the parameter block that are
overwritten from a symbol table before every launch (token counts of a nano-batch, request ranges,
number of attention work items, ...). Buffers never move, so an iteration is replayed by updating
the symbol table and walking the list. ``after_start`` dependencies express "do not start before X
has started" (used to force two kernels to be co-resident), the counterpart of
``OperatorWrapper::wait_for_start`` in the reference (pipeline/include/operatorWrapper.cuh:98-144).

The reference hand-writes this schedule in C++ for exactly two nano-batches
(pipeline/src/pipeline.cu:599-789); here it is data, built by :mod:`nanoflow_b200.runtime.pipeline`
from the JSON config, and executed either by the C++ executor (``_executor``) or by
:class:`PyExecutor` below (same semantics, for debugging and tests).
"""
from __future__ import annotations

import ctypes
from ctypes import (Structure, byref, c_float, c_int, c_longlong, c_void_p, sizeof)
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .. import ops as _ops

STREAM_CLASSES = ("gemm", "attn", "net", "other", "copy", "attn2", "net2")


class NormParams(Structure):
    _fields_ = [("out", c_void_p), ("x", c_void_p), ("w", c_void_p), ("resid", c_void_p),
                ("rows", c_int), ("cols", c_int), ("eps", c_float)]


class EmbeddingParams(Structure):
    _fields_ = [("out", c_void_p), ("table", c_void_p), ("host_ids", c_void_p), ("feedback_src", c_void_p),
                ("prev_tokens", c_void_p), ("ids_out", c_void_p), ("n_tokens", c_int), ("hidden", c_int),
                ("vocab", c_int), ("status", c_void_p)]


class GatherParams(Structure):
    _fields_ = [("out", c_void_p), ("inp", c_void_p), ("rows_idx", c_void_p), ("n", c_int), ("cols", c_int),
                ("ld_in", c_longlong), ("in_rows", c_int), ("status", c_void_p)]


class ArgmaxParams(Structure):
    _fields_ = [("idx_out", c_void_p), ("val_out", c_void_p), ("logits", c_void_p), ("rows", c_int),
                ("cols", c_int), ("ld", c_longlong), ("col_offset", c_int)]


class ArgmaxCombineParams(Structure):
    _fields_ = [("idx_out", c_void_p), ("cand_val", c_void_p), ("cand_idx", c_void_p), ("shards", c_int),
                ("rows", c_int)]


class CopyColsParams(Structure):
    _fields_ = [("out", c_void_p), ("ld_out", c_longlong), ("inp", c_void_p), ("ld_in", c_longlong),
                ("rows", c_int), ("cols", c_int)]


class MemcpyParams(Structure):
    _fields_ = [("dst", c_void_p), ("src", c_void_p), ("elem_bytes", c_longlong), ("count", c_int)]


class Memcpy2DParams(Structure):
    _fields_ = [("dst", c_void_p), ("src", c_void_p), ("dpitch", c_longlong), ("spitch", c_longlong),
                ("width", c_longlong), ("height", c_int)]


class SleepParams(Structure):
    _fields_ = [("micros", c_int)]


class KvMoveParams(Structure):
    _fields_ = [("pool", c_void_p), ("staging", c_void_p), ("page_ids", c_void_p), ("n_pages", c_int),
                ("page_bytes", c_longlong), ("num_pages", c_int), ("direction", c_int), ("num_ctas", c_int),
                ("status", c_void_p)]


GemmParams = _ops.GemmParams
RopeAppendParams = _ops.RopeAppendParams
RopeTableParams = _ops.RopeTableParams
AttnParams = _ops.AttnParams

KERNEL_OF = {
    GemmParams: "nfk_gemm_bf16", RopeAppendParams: "nfk_rope_append", RopeTableParams: "nfk_rope_table",
    NormParams: "nfk_norm_p",
    EmbeddingParams: "nfk_embedding_p", GatherParams: "nfk_gather_p", ArgmaxParams: "nfk_argmax_p",
    ArgmaxCombineParams: "nfk_argmax_combine_p", CopyColsParams: "nfk_copy_cols_p",
    MemcpyParams: "nfk_memcpy_p", Memcpy2DParams: "nfk_memcpy2d_p", KvMoveParams: "nfk_kv_move_p", SleepParams: "nfk_sleep_p",
}


@dataclass
class Op:
    name: str
    kernel: str                       # exported symbol
    params: Structure
    stream: str
    deps: List[int] = field(default_factory=list)         # wait for completion of these ops
    after_start: List[int] = field(default_factory=list)  # wait for the start of these ops
    gated: List[int] = field(default_factory=list)        # ops whose output this op consumes row block by row block
                                                          # behind device-side flags: launched once they have started
                                                          # (also listed in after_start), done only after they are done
    dyn: List[Tuple[str, str]] = field(default_factory=list)  # (int field of params, symbol name)
    layer: int = -1
    nano: int = -1


class OpGraph:
    def __init__(self) -> None:
        self.ops: List[Op] = []
        self.symbols: Dict[str, int] = {}

    def symbol(self, name: str) -> str:
        if name not in self.symbols:
            self.symbols[name] = len(self.symbols)
        return name

    def add(self, name: str, params: Structure, stream: str, deps: Sequence[Optional[int]] = (),
            dyn: Sequence[Tuple[str, str]] = (), kernel: Optional[str] = None,
            after_start: Sequence[Optional[int]] = (), layer: int = -1, nano: int = -1,
            gated: Sequence[Optional[int]] = ()) -> int:
        if stream not in STREAM_CLASSES:
            raise ValueError(f"unknown stream class {stream}")
        kernel = kernel or KERNEL_OF[type(params)]
        for f, s in dyn:
            self.symbol(s)
            if not hasattr(params, f):
                raise AttributeError(f"{type(params).__name__} has no field {f}")
        gated = sorted({d for d in gated if d is not None})
        op = Op(name=name, kernel=kernel, params=params, stream=stream,
                deps=sorted({d for d in deps if d is not None}),
                after_start=sorted({d for d in after_start if d is not None} | set(gated)), dyn=list(dyn),
                layer=layer, nano=nano, gated=gated)
        for d in op.deps + op.after_start:
            if not (0 <= d < len(self.ops)):
                raise ValueError(f"op {name}: dependency {d} is not an earlier op")
        self.ops.append(op)
        return len(self.ops) - 1

    # ---- static checks (the host-side dependency checker) -----------------------------------------
    def happens_before(self) -> List[set]:
        """For every op, the set of ops guaranteed to have completed before it starts
        (explicit deps plus stream order), transitively."""
        last_on_stream: Dict[str, int] = {}
        hb: List[set] = []
        for i, op in enumerate(self.ops):
            s = set()
            # a gated op cannot finish before the ops that feed it row block by row block have delivered
            # every block, so for the data those ops write the edge orders like a dependency
            preds = list(op.deps) + list(op.gated)
            if op.stream in last_on_stream:
                preds.append(last_on_stream[op.stream])
            for p in preds:
                s.add(p)
                s |= hb[p]
            hb.append(s)
            last_on_stream[op.stream] = i
        return hb


class PyExecutor:
    """Replays a graph from Python on torch streams (reference semantics for the C++ executor)."""

    def __init__(self, graph: OpGraph, single_stream: bool = False):
        import torch

        self.graph = graph
        self.torch = torch
        self.lib = _ops.lib()
        self.single_stream = single_stream
        self.streams = {c: torch.cuda.Stream() for c in STREAM_CLASSES}
        need_end = set()
        need_start = set()
        for op in graph.ops:
            need_end.update(op.deps)
            need_start.update(op.after_start)
        self.end_events = {i: torch.cuda.Event() for i in need_end}
        self.start_events = {i: torch.cuda.Event() for i in need_start}
        self.fns = [getattr(self.lib, op.kernel) for op in graph.ops]
        self.timing = False
        self.timeline: List[Tuple[str, str, float, float]] = []

    def run(self, symbols: Dict[str, int], main_stream=None) -> None:
        torch = self.torch
        main = main_stream or torch.cuda.current_stream()
        if not self.single_stream:
            fork = torch.cuda.Event()
            fork.record(main)
            for s in self.streams.values():
                s.wait_event(fork)
        tev = []
        for i, op in enumerate(self.graph.ops):
            st = main if self.single_stream else self.streams[op.stream]
            for f, sname in op.dyn:
                setattr(op.params, f, int(symbols[sname]))
            if not self.single_stream:
                for d in op.deps:
                    if self.graph.ops[d].stream != op.stream:
                        st.wait_event(self.end_events[d])
                for d in op.after_start:
                    st.wait_event(self.start_events[d])
            if i in self.start_events:
                self.start_events[i].record(st)
            if self.timing:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(st)
            rc = self.fns[i](byref(op.params), c_void_p(st.cuda_stream))
            if rc != 0:
                raise RuntimeError(f"op {op.name} ({op.kernel}): {_ops.ERRORS.get(rc, rc)}")
            if self.timing:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record(st)
                tev.append((op.name, op.stream, e0, e1))
            if i in self.end_events:
                self.end_events[i].record(st)
        if not self.single_stream:
            for s in self.streams.values():
                join = torch.cuda.Event()
                join.record(s)
                main.wait_event(join)
        if self.timing:
            torch.cuda.synchronize()
            base = tev[0][2] if tev else None
            self.timeline = [(n, s, base.elapsed_time(a) * 1e3, base.elapsed_time(b) * 1e3) for n, s, a, b in tev]
