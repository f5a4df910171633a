"""Plain PyTorch fp32 restatements of every kernel in :mod:`nanoflow_b200.ops`.

These are the oracles of the numerics tests and the building blocks of the CPU backend; they run on
any device and make no attempt to be fast. The paged-attention oracle plays the role of the
reference's ``cpu_reference::single_mha`` + ``append_paged_kv_cache`` (gemv/src/cpu_reference.h:47-167).
"""
from __future__ import annotations

from typing import Optional

import torch


def gemm(a, w, residual=None, beta=1.0, bias=None):
    out = a.float() @ w.float().t()
    if bias is not None:
        out = out + bias.float()
    if residual is not None:
        out = out + beta * residual.float()
    return out


def gemm_swiglu(a, w_gate, w_up):
    g = a.float() @ w_gate.float().t()
    u = a.float() @ w_up.float().t()
    return torch.nn.functional.silu(g) * u


def rmsnorm(x, w, eps):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def silu_mul(gate, up):
    return torch.nn.functional.silu(gate.float()) * up.float()


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """Rotary inverse frequencies, with Llama-3.1 style smoothing when ``scaling`` asks for it.

    The reference bakes the same smoothing into its kernel through constants derived in
    pipeline/include/config.h:101-110 and applied in pipeline/include/small_cuda_operator.cuh:36-44.
    """
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * torch.pi / inv
        smooth = (old / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        scaled = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
        inv = scaled
    return inv.float()


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, head_dim]; rotate-half convention (pairs i, i + head_dim/2)."""
    xf = x.float()
    ang = positions.to(x.device).float()[:, None] * inv_freq.to(x.device).float()[None, :]  # [T, hd/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    half = x.shape[-1] // 2
    lo, hi = xf[..., :half], xf[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def rope_append(qkv, kv_pool, inv_freq, positions, token_req, kv_indptr, kv_indices, *, q_heads,
                kv_heads, head_dim, q_off, k_off, v_off):
    """Returns rotated q [T, q_heads*hd] (fp32) and writes rotated k / v into kv_pool (in place)."""
    T = qkv.shape[0]
    page_size = kv_pool.shape[3]
    q = qkv[:, q_off:q_off + q_heads * head_dim].reshape(T, q_heads, head_dim)
    k = qkv[:, k_off:k_off + kv_heads * head_dim].reshape(T, kv_heads, head_dim)
    v = qkv[:, v_off:v_off + kv_heads * head_dim].reshape(T, kv_heads, head_dim)
    qr = rope(q, positions, inv_freq)
    kr = rope(k, positions, inv_freq)
    for t in range(T):
        b = int(token_req[t])
        pos = int(positions[t])
        page = int(kv_indices[int(kv_indptr[b]) + pos // page_size])
        slot = pos % page_size
        kv_pool[page, 0, :, slot, :] = kr[t].to(kv_pool.dtype)
        kv_pool[page, 1, :, slot, :] = v[t].to(kv_pool.dtype)
    return qr.reshape(T, q_heads * head_dim)


def gather_kv(kv_pool, kv_indptr, kv_indices, kv_last_page_len, b):
    """Contiguous K, V [kv_len, kv_heads, hd] (fp32) of request b from the paged pool."""
    pages = kv_indices[int(kv_indptr[b]):int(kv_indptr[b + 1])].long()
    page_size = kv_pool.shape[3]
    kv_len = (len(pages) - 1) * page_size + int(kv_last_page_len[b])
    k = kv_pool[pages, 0].permute(0, 2, 1, 3).reshape(-1, kv_pool.shape[2], kv_pool.shape[4])
    v = kv_pool[pages, 1].permute(0, 2, 1, 3).reshape(-1, kv_pool.shape[2], kv_pool.shape[4])
    return k[:kv_len].float(), v[:kv_len].float()


def paged_attention(q, kv_pool, qo_indptr, kv_indptr, kv_indices, kv_last_page_len, *, q_heads,
                    sm_scale=None, requests=None):
    """Causal attention of every query token against its request's paged KV.

    q: [T, q_heads*hd]. The last query token of request b sits at position kv_len-1.
    Returns fp32 [T, q_heads*hd]; rows of requests not in ``requests`` are left zero.
    """
    T = q.shape[0]
    kvh, hd = kv_pool.shape[2], kv_pool.shape[4]
    group = q_heads // kvh
    scale = sm_scale if sm_scale is not None else hd ** -0.5
    out = torch.zeros((T, q_heads * hd), dtype=torch.float32, device=q.device)
    B = len(qo_indptr) - 1
    for b in (requests if requests is not None else range(B)):
        t0, t1 = int(qo_indptr[b]), int(qo_indptr[b + 1])
        if t1 <= t0:
            continue
        k, v = gather_kv(kv_pool, kv_indptr, kv_indices, kv_last_page_len, b)
        kv_len = k.shape[0]
        qb = q[t0:t1].float().reshape(t1 - t0, q_heads, hd)
        kk = k.repeat_interleave(group, dim=1)  # [kv_len, q_heads, hd]
        vv = v.repeat_interleave(group, dim=1)
        s = torch.einsum("thd,khd->htk", qb, kk) * scale
        pos = kv_len - (t1 - t0) + torch.arange(t1 - t0, device=q.device)
        mask = torch.arange(kv_len, device=q.device)[None, :] <= pos[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[t0:t1] = torch.einsum("htk,khd->thd", p, vv).reshape(t1 - t0, q_heads * hd)
    return out


def argmax(logits, col_offset=0):
    return logits.float().argmax(dim=-1).int() + col_offset
