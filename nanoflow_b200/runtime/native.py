"""Python face of the C++ executor (``_executor`` extension module built from csrc/executor)."""
from __future__ import annotations

import ctypes
from typing import Dict, List

from .. import ops as _ops
from .graph import STREAM_CLASSES, OpGraph


def _load():
    from . import _executor  # noqa: WPS433  (built in-tree by nanoflow_b200.ops.build)
    return _executor


def load_host_module():
    """The host-only build of the executor (every CUDA runtime call logged instead of made); built
    on first use."""
    from ..ops import build
    build.build_executor_host()
    from . import _executor_host  # noqa: WPS433
    return _executor_host


class NativeExecutor:
    def __init__(self, graph: OpGraph, main_stream, single_stream: bool = False, device: int = 0,
                 use_cuda_graph: bool = False, host_only: bool = False):
        """``host_only``: drive the host-only build. No kernel runs; ``self.mod.host_log()`` lists the
        stream / event / graph calls the executor made (used by the CPU tests of the event wiring)."""
        mod = load_host_module() if host_only else _load()
        lib = None if host_only else _ops.lib()
        self.mod = mod
        self.graph = graph
        self.sym_names: List[str] = [None] * len(graph.symbols)
        for name, idx in graph.symbols.items():
            self.sym_names[idx] = name
        self.ex = mod.Executor(0 if host_only else int(main_stream.cuda_stream), int(device), bool(single_stream),
                               len(self.sym_names))
        for op in graph.ops:
            fn = mod.noop_fn() if host_only else ctypes.cast(getattr(lib, op.kernel), ctypes.c_void_p).value
            patches = []
            for f, s in op.dyn:
                desc = getattr(type(op.params), f)
                patches.append((desc.offset, graph.symbols[s], desc.size))
            self.ex.add_op(op.name, fn, bytes(op.params), STREAM_CLASSES.index(op.stream), list(op.deps),
                           list(op.after_start), patches)
        self.ex.freeze()
        # CUDA-graph mode: each iteration is captured, patched into the previous executable graph and
        # launched as one unit (see csrc/executor/executor.cpp)
        self.ex.set_graph_mode(bool(use_cuda_graph))
        self._keep = graph   # parameter blocks hold raw pointers into tensors owned by the engine

    def submit(self, symbols: Dict[str, int], timed: bool = False) -> int:
        return self.ex.submit([int(symbols[n]) for n in self.sym_names], timed)

    def wait(self, ticket: int) -> None:
        self.ex.wait(ticket)

    def timeline(self):
        return [(n, STREAM_CLASSES[c], a, b) for n, c, a, b in self.ex.timeline()]

    @property
    def launches(self) -> int:
        return self.ex.launches()

    @property
    def graph_stats(self):
        """(iterations launched as a CUDA graph, times the executable graph had to be rebuilt)."""
        return self.ex.graph_launches(), self.ex.graph_rebuilds()

    def close(self) -> None:
        self.ex.close()
