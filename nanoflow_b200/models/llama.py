"""Llama-family decoder (Llama-2/3/3.1, Qwen2 with QKV bias, Deepseek-LLM): weights, TP sharding, oracle.

* :class:`FullWeights` – unsharded Hugging Face layout (``[out, in]`` matrices), used by small
  models, the weight converter and the oracle.
* :class:`RankWeights` – what one GPU holds under tensor parallelism, in the layout the sm_100a
  kernels consume: every matrix ``[N, K]`` with K contiguous; QKV packed as K | V | Q rows (the
  order of the reference's ``KQV_l`` tensors, pipeline/utils/weightSaver.py:105-118); O and down
  projections split along K (their outputs are summed across GPUs), gate/up and QKV split along N;
  the LM head split along the vocabulary.
* :class:`ReferenceLlama` – plain PyTorch fp32 forward with a contiguous KV cache and greedy
  decoding: the correctness oracle of the engine (the role of groundtruth/test.py:12-38, which
  runs Hugging Face ``generate(top_k=1)`` and is compared by eye in the reference).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..config import ModelConfig
from ..ops import reference as ref


@dataclass
class FullLayer:
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    wg: torch.Tensor
    wu: torch.Tensor
    wd: torch.Tensor
    ln_attn: torch.Tensor
    ln_ffn: torch.Tensor
    bq: Optional[torch.Tensor] = None
    bk: Optional[torch.Tensor] = None
    bv: Optional[torch.Tensor] = None


@dataclass
class FullWeights:
    embed: torch.Tensor
    norm: torch.Tensor
    lm_head: torch.Tensor
    layers: List[FullLayer] = field(default_factory=list)


@dataclass
class LayerWeights:
    wqkv: torch.Tensor               # [kv_local*2 + q_local, hidden], rows K | V | Q
    wo: torch.Tensor                 # [hidden, q_local]
    wg: torch.Tensor                 # [ffn_local, hidden]
    wu: torch.Tensor                 # [ffn_local, hidden]
    wd: torch.Tensor                 # [hidden, ffn_local]
    ln_attn: torch.Tensor
    ln_ffn: torch.Tensor
    bqkv: Optional[torch.Tensor] = None
    # N-split form of the O projection, [hidden / tp, q_size]: rows rank*hidden/tp ... of the full matrix, for
    # nano-batches that all-gather the attention output instead of all-reducing the projection (the
    # reference's O1 weights, pipeline/src/vortexData.cu; only kept when a pipeline asks for it)
    wo1: Optional[torch.Tensor] = None


@dataclass
class RankWeights:
    embed: torch.Tensor              # [vocab, hidden] replicated
    norm: torch.Tensor
    lm_head: torch.Tensor            # [vocab_local, hidden] rows rank*vocab_local ...
    layers: List[LayerWeights]
    rank: int = 0
    tp: int = 1

    def to(self, device=None, dtype=None) -> "RankWeights":
        mv = lambda t: None if t is None else t.to(device=device, dtype=dtype)
        return RankWeights(mv(self.embed), mv(self.norm), mv(self.lm_head),
                           [LayerWeights(mv(l.wqkv), mv(l.wo), mv(l.wg), mv(l.wu), mv(l.wd), mv(l.ln_attn),
                                         mv(l.ln_ffn), mv(l.bqkv), mv(l.wo1)) for l in self.layers], self.rank, self.tp)

    def nbytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in (self.embed, self.norm, self.lm_head))
        for l in self.layers:
            for t in (l.wqkv, l.wo, l.wg, l.wu, l.wd, l.ln_attn, l.ln_ffn, l.bqkv, l.wo1):
                if t is not None:
                    n += t.numel() * t.element_size()
        return n


def random_full_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, dtype=torch.float32,
                        device="cpu") -> FullWeights:
    """N(0, std) matrices, norm weights 1 + N(0, std); deterministic in ``seed``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    rn = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype=dtype, device=device)
    h, f, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    fw = FullWeights(embed=rn(cfg.vocab_size, h), norm=(1 + rn(h)), lm_head=rn(cfg.vocab_size, h))
    for _ in range(cfg.num_layers):
        lay = FullLayer(wq=rn(cfg.num_q_heads * hd, h), wk=rn(cfg.num_kv_heads * hd, h),
                        wv=rn(cfg.num_kv_heads * hd, h), wo=rn(h, cfg.num_q_heads * hd),
                        wg=rn(f, h), wu=rn(f, h), wd=rn(h, f), ln_attn=1 + rn(h), ln_ffn=1 + rn(h))
        if cfg.qkv_bias:
            lay.bq, lay.bk, lay.bv = rn(cfg.num_q_heads * hd), rn(cfg.num_kv_heads * hd), rn(cfg.num_kv_heads * hd)
        fw.layers.append(lay)
    return fw


def shard_weights(fw: FullWeights, cfg: ModelConfig, rank: int, tp: int, dtype=torch.bfloat16,
                  device="cpu", o1: bool = False) -> RankWeights:
    """Slice the full model for one tensor-parallel rank (head-parallel attention, N-split gate/up,
    K-split O and down, vocab-split LM head). ``o1`` adds the N-split form of the O projection."""
    hd = cfg.head_dim
    ql, kl, fl = cfg.num_q_heads // tp * hd, cfg.num_kv_heads // tp * hd, cfg.intermediate_size // tp
    vl = ((cfg.vocab_size + tp - 1) // tp + 7) // 8 * 8
    mv = lambda t: t.to(dtype=dtype, device=device).contiguous()
    head = torch.zeros(vl, cfg.hidden_size, dtype=fw.lm_head.dtype)
    lo, hi = rank * vl, min(cfg.vocab_size, (rank + 1) * vl)
    if hi > lo:
        head[:hi - lo] = fw.lm_head[lo:hi]
    layers = []
    hs = cfg.hidden_size // tp
    for l in fw.layers:
        qs, ks = slice(rank * ql, (rank + 1) * ql), slice(rank * kl, (rank + 1) * kl)
        wqkv = torch.cat([l.wk[ks], l.wv[ks], l.wq[qs]], dim=0)
        bqkv = torch.cat([l.bk[ks], l.bv[ks], l.bq[qs]], dim=0) if l.bq is not None else None
        fs = slice(rank * fl, (rank + 1) * fl)
        layers.append(LayerWeights(wqkv=mv(wqkv), wo=mv(l.wo[:, qs]), wg=mv(l.wg[fs]), wu=mv(l.wu[fs]),
                                   wd=mv(l.wd[:, fs]), ln_attn=mv(l.ln_attn), ln_ffn=mv(l.ln_ffn),
                                   bqkv=None if bqkv is None else mv(bqkv),
                                   wo1=mv(l.wo[rank * hs:(rank + 1) * hs]) if (o1 and tp > 1) else None))
    return RankWeights(embed=mv(fw.embed), norm=mv(fw.norm), lm_head=mv(head), layers=layers, rank=rank, tp=tp)


def random_rank_weights(cfg: ModelConfig, rank: int, tp: int, device, dtype=torch.bfloat16, seed: int = 0,
                        std: float = 0.02, o1: bool = False) -> RankWeights:
    """Random-init shard generated directly on ``device`` (never materialises the full model):
    the ``--empty_weight`` path of the reference (pipeline/src/vortexData.cu:386-406) with defined
    values instead of uninitialised memory."""
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)

    def rn(*shape):
        t = torch.empty(*shape, dtype=dtype, device=device)
        t.normal_(0.0, std, generator=g)
        return t

    def ones(n):
        t = rn(n)
        t += 1
        return t

    h, hd = cfg.hidden_size, cfg.head_dim
    ql, kl, fl = cfg.num_q_heads // tp * hd, cfg.num_kv_heads // tp * hd, cfg.intermediate_size // tp
    vl = ((cfg.vocab_size + tp - 1) // tp + 7) // 8 * 8
    # replicated tensors must agree across ranks: draw them from a rank-independent stream
    g_shared = torch.Generator(device=device).manual_seed(seed * 1000 + 999)
    embed = torch.empty(cfg.vocab_size, h, dtype=dtype, device=device).normal_(0.0, std, generator=g_shared)
    norm = torch.empty(h, dtype=dtype, device=device).normal_(0.0, std, generator=g_shared) + 1
    layers = []
    for _ in range(cfg.num_layers):
        ln_a = torch.empty(h, dtype=dtype, device=device).normal_(0.0, std, generator=g_shared) + 1
        ln_f = torch.empty(h, dtype=dtype, device=device).normal_(0.0, std, generator=g_shared) + 1
        layers.append(LayerWeights(wqkv=rn(ql + 2 * kl, h), wo=rn(h, ql), wg=rn(fl, h), wu=rn(fl, h),
                                   wd=rn(h, fl), ln_attn=ln_a, ln_ffn=ln_f,
                                   bqkv=rn(ql + 2 * kl) if cfg.qkv_bias else None,
                                   wo1=rn(h // tp, cfg.num_q_heads * hd) if (o1 and tp > 1) else None))
    return RankWeights(embed=embed, norm=norm, lm_head=rn(vl, h), layers=layers, rank=rank, tp=tp)


class ReferenceLlama:
    """fp32 oracle: full-sequence forward and greedy generation with a contiguous KV cache."""

    def __init__(self, cfg: ModelConfig, weights: FullWeights):
        self.cfg = cfg
        self.w = weights
        self.inv_freq = ref.rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)

    def _layer(self, x, lay: FullLayer, positions, cache):
        cfg = self.cfg
        T = x.shape[0]
        hd = cfg.head_dim
        h = ref.rmsnorm(x, lay.ln_attn, cfg.rms_norm_eps)
        q = h @ lay.wq.float().t()
        k = h @ lay.wk.float().t()
        v = h @ lay.wv.float().t()
        if lay.bq is not None:
            q, k, v = q + lay.bq.float(), k + lay.bk.float(), v + lay.bv.float()
        q = ref.rope(q.reshape(T, cfg.num_q_heads, hd), positions, self.inv_freq)
        k = ref.rope(k.reshape(T, cfg.num_kv_heads, hd), positions, self.inv_freq)
        v = v.reshape(T, cfg.num_kv_heads, hd)
        if cache["k"] is None:
            cache["k"], cache["v"] = k, v
        else:
            cache["k"], cache["v"] = torch.cat([cache["k"], k]), torch.cat([cache["v"], v])
        kk = cache["k"].repeat_interleave(cfg.group_size, dim=1)
        vv = cache["v"].repeat_interleave(cfg.group_size, dim=1)
        s = torch.einsum("thd,khd->htk", q, kk) * hd ** -0.5
        kv_len = kk.shape[0]
        mask = torch.arange(kv_len)[None, :] <= positions[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("htk,khd->thd", torch.softmax(s, -1), vv).reshape(T, -1)
        x = x + o @ lay.wo.float().t()
        h = ref.rmsnorm(x, lay.ln_ffn, cfg.rms_norm_eps)
        act = torch.nn.functional.silu(h @ lay.wg.float().t()) * (h @ lay.wu.float().t())
        return x + act @ lay.wd.float().t()

    def forward(self, tokens: torch.Tensor, caches=None, start: int = 0):
        """tokens [T] of one sequence starting at position ``start``; returns logits [T, vocab]."""
        cfg = self.cfg
        if caches is None:
            caches = [dict(k=None, v=None) for _ in range(cfg.run_layers)]
        x = self.w.embed.float()[tokens.long()]
        positions = start + torch.arange(tokens.numel())
        for l in range(cfg.run_layers):
            x = self._layer(x, self.w.layers[l % cfg.num_layers], positions, caches[l])
        x = ref.rmsnorm(x, self.w.norm, cfg.rms_norm_eps)
        return x @ self.w.lm_head.float().t(), caches

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos_token_id: Optional[int] = None,
                 return_logits: bool = False):
        toks = torch.tensor(list(prompt), dtype=torch.long)
        logits, caches = self.forward(toks)
        out, all_logits = [], []
        pos = toks.numel()
        nxt = int(logits[-1].argmax())
        all_logits.append(logits[-1])
        out.append(nxt)
        while len(out) < max_new_tokens and (eos_token_id is None or nxt != eos_token_id):
            logits, caches = self.forward(torch.tensor([nxt]), caches, start=pos)
            pos += 1
            nxt = int(logits[-1].argmax())
            all_logits.append(logits[-1])
            out.append(nxt)
        return (out, torch.stack(all_logits)) if return_logits else out
