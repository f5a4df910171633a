"""Python entry points for the sm_100a kernel library (``libnanoflow_kernels.so``).

Each function takes torch CUDA tensors, checks what the C ABI cannot (dtype, device, contiguity),
and launches on the current torch stream through ``ctypes``. There is no PyTorch fallback: if the
library is missing or a launcher rejects its arguments a ``RuntimeError`` is raised. Plain PyTorch
fp32 restatements of every op live in :mod:`nanoflow_b200.ops.reference` and are used by the tests
and by the CPU oracle only.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p, POINTER, Structure, byref
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libnanoflow_kernels.so"
_lib = None

ERRORS = {1: "bad argument (shape / alignment / size limit)", 2: "CUDA call failed",
          3: "unsupported configuration"}

STATUS_CODES = {
    0x100: "timeout waiting for a TMA stage", 0x200: "timeout waiting for a free smem stage",
    0x300: "timeout waiting for an accumulator", 0x400: "timeout waiting for a free accumulator",
    0x500: "timeout waiting for a peer flag", 0x600: "timeout in a grid barrier",
    0x700: "out-of-range index skipped",
}


class GemmParams(Structure):
    _fields_ = [("A", c_void_p), ("B", c_void_p), ("B2", c_void_p), ("D", c_void_p),
                ("C", c_void_p), ("bias", c_void_p),
                ("lda", c_longlong), ("ldb", c_longlong), ("ldd", c_longlong), ("ldc", c_longlong),
                ("beta", c_float), ("M", c_int), ("N", c_int), ("K", c_int),
                ("epilogue", c_int), ("tile_n", c_int), ("num_ctas", c_int),
                ("status", c_void_p), ("tile_m", c_int), ("split_k", c_int), ("workspace", c_void_p),
                ("workspace_bytes", c_longlong),
                ("rs_heap", c_void_p * 8), ("rs_rank", c_int), ("rs_nranks", c_int), ("rs_slab_off", c_longlong),
                ("rs_rows_cap", c_int), ("rs_flag_off", c_longlong), ("rs_epoch", c_int), ("smem_budget_kb", c_int),
                ("cta_group", c_int), ("stream_k", c_int),
                ("norm_w", c_void_p), ("norm_out", c_void_p), ("norm_ld", c_longlong), ("norm_eps", c_float),
                ("rs_staged", c_int), ("gate_flags", c_void_p), ("gate_epoch", c_int), ("gate_nranks", c_int)]


class RopeAppendParams(Structure):
    _fields_ = [("qkv", c_void_p), ("ld_qkv", c_longlong),
                ("q_off", c_int), ("k_off", c_int), ("v_off", c_int),
                ("q_out", c_void_p), ("kv_pool", c_void_p), ("inv_freq", c_void_p),
                ("positions", c_void_p), ("token_req", c_void_p), ("kv_indptr", c_void_p),
                ("kv_indices", c_void_p),
                ("T", c_int), ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int),
                ("page_size", c_int), ("num_pages", c_int), ("status", c_void_p), ("cos_sin", c_void_p)]


class RopeTableParams(Structure):
    _fields_ = [("cos_sin", c_void_p), ("inv_freq", c_void_p), ("positions", c_void_p), ("T", c_int),
                ("half", c_int)]


class AttnParams(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("kv_pool", c_void_p),
                ("qo_indptr", c_void_p), ("kv_indptr", c_void_p), ("kv_indices", c_void_p),
                ("kv_last_page_len", c_void_p),
                ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int),
                ("page_size", c_int), ("num_pages", c_int), ("sm_scale", c_float),
                ("num_ctas", c_int), ("req_begin", c_int), ("req_count", c_int),
                ("chunk_pages", c_int), ("workspace", c_void_p), ("max_chunks", c_int),
                ("items", c_void_p), ("num_items", c_int), ("status", c_void_p), ("decode_stages", c_int)]


def library_path() -> Path:
    return _LIB_PATH


def lib():
    """Load the kernel library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m nanoflow_b200.ops.build` "
                "(the CUDA kernels have no PyTorch fallback)")
        _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {ERRORS.get(rc, rc)}")


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _bf16(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA bf16 tensor")


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous CUDA int32 tensor")


def new_status(device=None) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device or "cuda")


def sm_count(device=None) -> int:
    """SMs of ``device`` (the current CUDA device by default); a B200's 148 on a machine without a GPU,
    where graphs are only built for analysis."""
    if not torch.cuda.is_available():
        return 148
    if device is not None and torch.device(device).type != "cuda":
        return 148
    return int(torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
               .multi_processor_count)


def check_status(status: torch.Tensor, what: str = "kernel") -> None:
    """Read a device status word (synchronises) and raise if a kernel reported a problem."""
    code = int(status.item()) & 0xFFFFFFFF
    if code:
        status.zero_()
        raise RuntimeError(f"{what}: device status 0x{code:x} ({STATUS_CODES.get(code & 0xF00, '?')})")


# ------------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, beta: float = 1.0,
         bias: Optional[torch.Tensor] = None, tile_n: int = 0, num_ctas: int = 0,
         status: Optional[torch.Tensor] = None, tile_m: int = 0, split_k: int = 0,
         workspace: Optional[torch.Tensor] = None, smem_budget_kb: int = 0,
         cta_group: int = 0, stream_k: int = 0, norm_w: Optional[torch.Tensor] = None,
         norm_out: Optional[torch.Tensor] = None, norm_eps: float = 1e-5,
         gate_flags: Optional[torch.Tensor] = None, gate_epoch: int = 0, gate_nranks: int = 1) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) (+ beta * residual). Rows may be strided.

    With ``norm_w`` / ``norm_out`` the call also leaves ``norm_out = RMSNorm(out) * norm_w`` (from the
    split-K reduce pass when K is split, by a norm launch otherwise).

    ``tile_n`` / ``tile_m`` / ``split_k`` pin the kernel shape (0 = let the launcher's cost model
    choose); split-K needs ``workspace`` (any dtype, >= split_k*M*N*4 bytes).

    ``gate_flags`` (int32 [ceil(M/128), 8]): rows of ``a`` are still arriving; the kernel waits, per
    128-row block, until words [block, 0:gate_nranks] have reached ``gate_epoch``."""
    _bf16(a, "a"); _bf16(w, "w")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or a.stride(1) != 1 or w.stride(1) != 1:
        raise RuntimeError("gemm: inner dimensions must match and be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _bf16(out, "out")
    if out.shape != (M, N) or out.stride(1) != 1:
        raise RuntimeError("gemm: bad out")
    p = GemmParams()
    p.A, p.B, p.B2, p.D = _p(a), _p(w), c_void_p(0), _p(out)
    p.C, p.bias = _p(residual), _p(bias)
    p.lda, p.ldb, p.ldd = a.stride(0), w.stride(0), out.stride(0)
    p.ldc = residual.stride(0) if residual is not None else 0
    if residual is not None:
        _bf16(residual, "residual")
        if residual.shape != (M, N) or residual.stride(1) != 1:
            raise RuntimeError("gemm: bad residual")
    if bias is not None:
        _bf16(bias, "bias")
        if bias.numel() != N or not bias.is_contiguous():
            raise RuntimeError("gemm: bad bias")
    p.beta, p.M, p.N, p.K = beta, M, N, K
    p.epilogue, p.tile_n, p.num_ctas = 0, tile_n, num_ctas
    p.status = _p(status)
    p.tile_m, p.split_k = tile_m, split_k
    p.workspace = _p(workspace)
    p.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    p.smem_budget_kb = smem_budget_kb
    p.cta_group = cta_group
    p.stream_k = stream_k
    if norm_w is not None:
        _bf16(norm_w, "norm_w"); _bf16(norm_out, "norm_out")
        p.norm_w, p.norm_out, p.norm_ld, p.norm_eps = _p(norm_w), _p(norm_out), norm_out.stride(0), norm_eps
    _set_gate(p, gate_flags, gate_epoch, gate_nranks, M)
    _check(lib().nfk_gemm_bf16(byref(p), _stream()), "nfk_gemm_bf16")
    return out


def _set_gate(p: "GemmParams", flags: Optional[torch.Tensor], epoch: int, nranks: int, M: int) -> None:
    if flags is None:
        return
    _i32(flags, "gate_flags")
    if not flags.is_contiguous() or flags.numel() < (M + 127) // 128 * 8:
        raise RuntimeError("gemm: gate_flags must be a contiguous int32 [ceil(M/128), 8] tensor")
    p.gate_flags, p.gate_epoch, p.gate_nranks = _p(flags), epoch, nranks


class GemmPlan(Structure):
    _fields_ = [("tile_n", c_int), ("tile_m", c_int), ("cta_group", c_int), ("split_k", c_int), ("stream_k", c_int),
                ("tiles", c_int), ("workers", c_int), ("num_kb", c_int),
                ("tail_first_tile", c_int), ("tail_range_kb", c_int), ("tail_max_pieces", c_int),
                ("stages", c_int), ("smem_bytes", c_int)]


def gemm_plan(M: int, N: int, K: int, *, swiglu: bool = False, tile_n: int = 0, tile_m: int = 0, cta_group: int = 0,
              split_k: int = 0, stream_k: int = 0, num_ctas: int = 0, workspace_bytes: int = 0,
              smem_budget_kb: int = 0) -> dict:
    """What ``gemm`` / ``gemm_swiglu`` would launch for these sizes (tile shape, tiles, workers, stream-K
    tail) without launching anything; works without a GPU. ``workspace_bytes`` > 0 stands for a caller
    that passes a workspace of that size."""
    p = GemmParams()
    p.M, p.N, p.K = M, N, K
    p.epilogue, p.tile_n, p.tile_m, p.cta_group = (1 if swiglu else 0), tile_n, tile_m, cta_group
    p.split_k, p.stream_k, p.num_ctas, p.smem_budget_kb = split_k, stream_k, num_ctas, smem_budget_kb
    if workspace_bytes > 0:
        p.workspace, p.workspace_bytes = c_void_p(256), workspace_bytes    # never dereferenced by the planner
    out = GemmPlan()
    _check(lib().nfk_gemm_describe(byref(p), byref(out)), "nfk_gemm_describe")
    return {f: getattr(out, f) for f, _ in GemmPlan._fields_}


def gemm_swiglu(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *,
                out: Optional[torch.Tensor] = None, tile_n: int = 0, num_ctas: int = 0,
                status: Optional[torch.Tensor] = None, tile_m: int = 0, split_k: int = 0,
                workspace: Optional[torch.Tensor] = None, cta_group: int = 0,
                stream_k: int = 0, smem_budget_kb: int = 0, gate_flags: Optional[torch.Tensor] = None,
                gate_epoch: int = 0, gate_nranks: int = 1) -> torch.Tensor:
    """out[M,F] = silu(a @ w_gate^T) * (a @ w_up^T), gate and up products fused in one kernel.
    ``gate_flags``: as in :func:`gemm`."""
    _bf16(a, "a"); _bf16(w_gate, "w_gate"); _bf16(w_up, "w_up")
    M, K = a.shape
    F, K2 = w_gate.shape
    if w_up.shape != w_gate.shape or K != K2 or w_up.stride(0) != w_gate.stride(0):
        raise RuntimeError("gemm_swiglu: gate/up shapes must match")
    if a.stride(1) != 1 or w_gate.stride(1) != 1 or w_up.stride(1) != 1:
        raise RuntimeError("gemm_swiglu: inner dimension must be contiguous")
    if out is None:
        out = torch.empty((M, F), dtype=torch.bfloat16, device=a.device)
    p = GemmParams()
    p.A, p.B, p.B2, p.D = _p(a), _p(w_gate), _p(w_up), _p(out)
    p.C, p.bias = c_void_p(0), c_void_p(0)
    p.lda, p.ldb, p.ldd, p.ldc = a.stride(0), w_gate.stride(0), out.stride(0), 0
    p.beta, p.M, p.N, p.K = 0.0, M, F, K
    p.epilogue, p.tile_n, p.num_ctas = 1, tile_n, num_ctas
    p.status = _p(status)
    p.tile_m, p.split_k = tile_m, split_k
    p.workspace = _p(workspace)
    p.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    p.cta_group = cta_group
    p.stream_k = stream_k
    p.smem_budget_kb = smem_budget_kb
    _set_gate(p, gate_flags, gate_epoch, gate_nranks, M)
    _check(lib().nfk_gemm_bf16(byref(p), _stream()), "nfk_gemm_bf16(swiglu)")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None):
    _bf16(x, "x"); _bf16(w, "w")
    if not x.is_contiguous():
        raise RuntimeError("rmsnorm: x must be contiguous")
    rows, cols = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().nfk_rmsnorm(_p(out), _p(x), _p(w), c_int(rows), c_int(cols), c_float(eps),
                             _stream()), "nfk_rmsnorm")
    return out


def add_rmsnorm(resid: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None):
    """resid += x (in place); returns rmsnorm(resid)."""
    _bf16(x, "x"); _bf16(w, "w"); _bf16(resid, "resid")
    if not (x.is_contiguous() and resid.is_contiguous()) or x.shape != resid.shape:
        raise RuntimeError("add_rmsnorm: contiguous tensors of one shape expected")
    rows, cols = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().nfk_add_rmsnorm(_p(out), _p(resid), _p(x), _p(w), c_int(rows), c_int(cols),
                                 c_float(eps), _stream()), "nfk_add_rmsnorm")
    return out


def embedding(table: torch.Tensor, host_ids: Optional[torch.Tensor], *,
              feedback_src: Optional[torch.Tensor] = None,
              prev_tokens: Optional[torch.Tensor] = None, ids_out: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    _bf16(table, "table")
    ref = host_ids if host_ids is not None else feedback_src
    n = ref.numel()
    vocab, hidden = table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.bfloat16, device=table.device)
    for t, nm in ((host_ids, "host_ids"), (feedback_src, "feedback_src"), (prev_tokens, "prev_tokens"),
                  (ids_out, "ids_out")):
        if t is not None:
            _i32(t, nm)
    _check(lib().nfk_embedding(_p(out), _p(table), _p(host_ids), _p(feedback_src), _p(prev_tokens),
                               _p(ids_out), c_int(n), c_int(hidden), c_int(vocab), _p(status),
                               _stream()), "nfk_embedding")
    return out


def gather_rows(x: torch.Tensor, rows_idx: torch.Tensor, out: Optional[torch.Tensor] = None,
                status: Optional[torch.Tensor] = None):
    _bf16(x, "x"); _i32(rows_idx, "rows_idx")
    n, cols = rows_idx.numel(), x.shape[1]
    if x.stride(1) != 1:
        raise RuntimeError("gather_rows: rows must be contiguous")
    if out is None:
        out = torch.empty((n, cols), dtype=torch.bfloat16, device=x.device)
    _check(lib().nfk_gather_rows(_p(out), _p(x), _p(rows_idx), c_int(n), c_int(cols),
                                 c_longlong(x.stride(0)), _p(status), c_int(x.shape[0]), _stream()),
           "nfk_gather_rows")
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None):
    _bf16(gate, "gate"); _bf16(up, "up")
    if not (gate.is_contiguous() and up.is_contiguous()):
        raise RuntimeError("silu_mul: contiguous tensors expected")
    if out is None:
        out = torch.empty_like(gate)
    _check(lib().nfk_silu_mul(_p(out), _p(gate), _p(up), c_longlong(gate.numel()), _stream()),
           "nfk_silu_mul")
    return out


def copy_cols(dst: torch.Tensor, src: torch.Tensor):
    """dst[:, :] = src[:, :] for 2-D views with unit inner stride (column-block extract/insert)."""
    _bf16(dst, "dst"); _bf16(src, "src")
    if dst.shape != src.shape or dst.stride(1) != 1 or src.stride(1) != 1:
        raise RuntimeError("copy_cols: shapes must match, inner stride 1")
    _check(lib().nfk_copy_cols(_p(dst), c_longlong(dst.stride(0)), _p(src), c_longlong(src.stride(0)),
                               c_int(src.shape[0]), c_int(src.shape[1]), _stream()), "nfk_copy_cols")
    return dst


def transpose(x: torch.Tensor, out: Optional[torch.Tensor] = None):
    _bf16(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("transpose: contiguous input expected")
    r, c = x.shape
    if out is None:
        out = torch.empty((c, r), dtype=torch.bfloat16, device=x.device)
    _check(lib().nfk_transpose(_p(out), _p(x), c_int(r), c_int(c), _stream()), "nfk_transpose")
    return out


def argmax(logits: torch.Tensor, *, col_offset: int = 0, idx_out: Optional[torch.Tensor] = None,
           val_out: Optional[torch.Tensor] = None):
    _bf16(logits, "logits")
    rows, cols = logits.shape
    if logits.stride(1) != 1:
        raise RuntimeError("argmax: rows must be contiguous")
    if idx_out is None:
        idx_out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib().nfk_argmax(_p(idx_out), _p(val_out), _p(logits), c_int(rows), c_int(cols),
                            c_longlong(logits.stride(0)), c_int(col_offset), _stream()), "nfk_argmax")
    return idx_out


def argmax_combine(cand_val: torch.Tensor, cand_idx: torch.Tensor,
                   idx_out: Optional[torch.Tensor] = None):
    shards, rows = cand_val.shape
    if cand_val.dtype != torch.float32 or not cand_val.is_contiguous():
        raise RuntimeError("argmax_combine: cand_val must be contiguous fp32")
    _i32(cand_idx, "cand_idx")
    if idx_out is None:
        idx_out = torch.empty(rows, dtype=torch.int32, device=cand_val.device)
    _check(lib().nfk_argmax_combine(_p(idx_out), _p(cand_val), _p(cand_idx), c_int(shards),
                                    c_int(rows), _stream()), "nfk_argmax_combine")
    return idx_out


def sleep_us(micros: int):
    _check(lib().nfk_sleep(c_int(micros), _stream()), "nfk_sleep")


def flag_add(flag: torch.Tensor, v: int = 1):
    _check(lib().nfk_flag_add(_p(flag), ctypes.c_uint(v), _stream()), "nfk_flag_add")


def flag_clear(flag: torch.Tensor):
    _check(lib().nfk_flag_clear(_p(flag), _stream()), "nfk_flag_clear")


def flag_wait(flag: torch.Tensor, target: int, timeout_us: int, status: Optional[torch.Tensor] = None):
    _check(lib().nfk_flag_wait(_p(flag), ctypes.c_uint(target), c_int(timeout_us), _p(status),
                               _stream()), "nfk_flag_wait")


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, kv_pool: torch.Tensor,
                inv_freq: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor,
                kv_indptr: torch.Tensor, kv_indices: torch.Tensor, *, q_heads: int, kv_heads: int,
                head_dim: int, q_off: int, k_off: int, v_off: int,
                status: Optional[torch.Tensor] = None, cos_sin: Optional[torch.Tensor] = None):
    """Rotate q/k, write q to q_out and k/v into their page slots (see csrc/kernels/rope_append.cu).

    kv_pool: [num_pages, 2, kv_heads, page_size, head_dim] bf16 (one layer).
    """
    _bf16(qkv, "qkv"); _bf16(q_out, "q_out"); _bf16(kv_pool, "kv_pool")
    for t, nm in ((positions, "positions"), (token_req, "token_req"), (kv_indptr, "kv_indptr"),
                  (kv_indices, "kv_indices")):
        _i32(t, nm)
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise RuntimeError("rope_append: inv_freq must be fp32 [head_dim/2]")
    num_pages, two, kvh, page_size, hd = kv_pool.shape
    if two != 2 or kvh != kv_heads or hd != head_dim or not kv_pool.is_contiguous():
        raise RuntimeError("rope_append: kv_pool must be contiguous [pages,2,kv_heads,page,head_dim]")
    p = RopeAppendParams()
    p.qkv, p.ld_qkv = _p(qkv), qkv.stride(0)
    p.q_off, p.k_off, p.v_off = q_off, k_off, v_off
    p.q_out, p.kv_pool, p.inv_freq = _p(q_out), _p(kv_pool), _p(inv_freq)
    p.positions, p.token_req = _p(positions), _p(token_req)
    p.kv_indptr, p.kv_indices = _p(kv_indptr), _p(kv_indices)
    p.T, p.q_heads, p.kv_heads, p.head_dim = qkv.shape[0], q_heads, kv_heads, head_dim
    p.page_size, p.num_pages = page_size, num_pages
    p.status = _p(status)
    if cos_sin is not None:
        if cos_sin.dtype != torch.float32 or cos_sin.numel() < qkv.shape[0] * head_dim or not cos_sin.is_contiguous():
            raise RuntimeError("rope_append: cos_sin must be contiguous fp32 [T, head_dim/2, 2]")
        p.cos_sin = _p(cos_sin)
    _check(lib().nfk_rope_append(byref(p), _stream()), "nfk_rope_append")


def rope_table(inv_freq: torch.Tensor, positions: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[T, head_dim/2, 2] fp32 (cos, sin) of positions[t] * inv_freq[i]: the angles every layer's
    rope_append of one iteration shares."""
    _i32(positions, "positions")
    T, half = positions.numel(), inv_freq.numel()
    if out is None:
        out = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    p = RopeTableParams()
    p.cos_sin, p.inv_freq, p.positions, p.T, p.half = _p(out), _p(inv_freq), _p(positions), T, half
    _check(lib().nfk_rope_table(byref(p), _stream()), "nfk_rope_table")
    return out


def _attn_common(q, out, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, q_heads,
                 sm_scale, num_ctas, status) -> AttnParams:
    _bf16(q, "q"); _bf16(out, "out"); _bf16(kv_pool, "kv_pool")
    for t, nm in ((qo_indptr, "qo_indptr"), (kv_indptr, "kv_indptr"), (kv_indices, "kv_indices"),
                  (kv_last_page_len, "kv_last_page_len")):
        _i32(t, nm)
    num_pages, two, kv_heads, page_size, hd = kv_pool.shape
    if not (q.is_contiguous() and out.is_contiguous() and kv_pool.is_contiguous()):
        raise RuntimeError("attention: contiguous q/out/kv_pool expected")
    p = AttnParams()
    p.q, p.out, p.kv_pool = _p(q), _p(out), _p(kv_pool)
    p.qo_indptr, p.kv_indptr, p.kv_indices = _p(qo_indptr), _p(kv_indptr), _p(kv_indices)
    p.kv_last_page_len = _p(kv_last_page_len)
    p.q_heads, p.kv_heads, p.head_dim = q_heads, kv_heads, hd
    p.page_size, p.num_pages = page_size, num_pages
    p.sm_scale = sm_scale if sm_scale is not None else hd ** -0.5
    p.num_ctas = num_ctas
    p.status = _p(status)
    return p


def attn_decode(q, out, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, *,
                q_heads: int, req_begin: int, req_count: int, sm_scale: Optional[float] = None,
                num_ctas: int = 0, chunk_pages: int = 0, workspace: Optional[torch.Tensor] = None,
                max_chunks: int = 1, status: Optional[torch.Tensor] = None, stages: int = 0, impl: str = ""):
    """Single-query attention for requests [req_begin, req_begin+req_count) over the paged pool.
    ``stages``: pages in flight per warp, 3 (default) or 2 (64 KB of shared memory per CTA instead of 96).
    ``impl``: "" = per-warp cp.async rings, "tma" = pages copied by a TMA producer warp (head_dim 128;
    ``stages`` may then also be 4)."""
    p = _attn_common(q, out, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, q_heads,
                     sm_scale, num_ctas, status)
    p.decode_stages = stages
    p.req_begin, p.req_count = req_begin, req_count
    p.chunk_pages, p.max_chunks = chunk_pages, max_chunks
    p.workspace = _p(workspace)
    if chunk_pages > 0:
        need = req_count * q_heads * max_chunks * (kv_pool.shape[-1] + 2)
        if workspace is None or workspace.dtype != torch.float32 or workspace.numel() < need:
            raise RuntimeError("attn_decode: split-KV needs an fp32 workspace of "
                               f"{need} elements")
    if impl == "tma":
        _check(lib().nfk_attn_decode_tma(byref(p), _stream()), "nfk_attn_decode_tma")
    else:
        _check(lib().nfk_attn_decode(byref(p), _stream()), "nfk_attn_decode")
    return out


def attn_prefill(q, out, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, items, *,
                 q_heads: int, sm_scale: Optional[float] = None, num_ctas: int = 0,
                 status: Optional[torch.Tensor] = None, impl: str = "auto"):
    """Causal attention for work items [(request, first token, token count)] over the paged pool.

    ``impl``: "ws" = warp-specialised tcgen05 kernel (head_dim 128), "tc" = the earlier tcgen05 kernel,
    "mma" = warp-level mma.sync kernel, "auto" = ws when the head size allows."""
    p = _attn_common(q, out, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, q_heads,
                     sm_scale, num_ctas, status)
    _i32(items, "items")
    p.items, p.num_items = _p(items), items.shape[0]
    if impl == "ws" or (impl == "auto" and kv_pool.shape[-1] == 128):
        _check(lib().nfk_attn_prefill_ws(byref(p), _stream()), "nfk_attn_prefill_ws")
    elif impl == "tc":
        _check(lib().nfk_attn_prefill_tc(byref(p), _stream()), "nfk_attn_prefill_tc")
    else:
        _check(lib().nfk_attn_prefill(byref(p), _stream()), "nfk_attn_prefill")
    return out


def kv_move_pages(pool: torch.Tensor, staging: torch.Tensor, page_ids: torch.Tensor, *,
                  to_staging: bool, num_ctas: int = 8, status: Optional[torch.Tensor] = None):
    """Gather (to_staging) or scatter whole pages between a layer pool and a staging buffer."""
    _i32(page_ids, "page_ids")
    num_pages = pool.shape[0]
    page_bytes = pool[0].numel() * pool.element_size()
    n = page_ids.numel()
    if staging.numel() * staging.element_size() < n * page_bytes:
        raise RuntimeError("kv_move_pages: staging buffer too small")
    _check(lib().nfk_kv_move_pages(_p(pool), _p(staging), _p(page_ids), c_int(n),
                                   c_longlong(page_bytes), c_int(num_pages),
                                   c_int(0 if to_staging else 1), c_int(num_ctas), _p(status),
                                   _stream()), "nfk_kv_move_pages")
