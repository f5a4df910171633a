"""CPU backend: executes a scheduler :class:`BatchPlan` with plain PyTorch fp32 ops.

It follows exactly the data flow of the GPU engine (device-side token feedback through
``feedback_src``, paged KV pool with the same layout, decode-first token order, nano-batch cuts,
tensor-parallel shards whose partial O / down products are summed and whose vocab-sharded arg-max
candidates are combined) so the scheduler, the async control flow and the sharding maths can be
tested end to end without a GPU, against :class:`nanoflow_b200.models.ReferenceLlama`.
All ranks of a TP group run inside this one object.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..config import NanoflowConfig
from ..models.llama import RankWeights
from ..ops import reference as ref
from ..serving.scheduler import BatchPlan


class CpuEngine:
    def __init__(self, cfg: NanoflowConfig, rank_weights: List[RankWeights], num_pages: int = 256):
        self.cfg, self.model, self.eng = cfg, cfg.model, cfg.engine
        self.ranks = [w.to(dtype=torch.float32) for w in rank_weights]
        self.tp = len(rank_weights)
        m = self.model
        self.num_pages = num_pages
        self.kv_pool = [[torch.zeros(num_pages, 2, m.num_kv_heads // self.tp, self.eng.page_size, m.head_dim)
                         for _ in range(m.run_layers)] for _ in range(self.tp)]
        self.inv_freq = ref.rope_inv_freq(m.head_dim, m.rope_theta, m.rope_scaling)
        self.sampled = torch.zeros(self.eng.max_batch_size, dtype=torch.int32)
        self._staged: Optional[BatchPlan] = None
        self._inflight: List[np.ndarray] = []
        self._last = np.zeros(0, dtype=np.int32)
        self.last_logits: Optional[torch.Tensor] = None

    def update(self, plan: BatchPlan) -> None:
        self._staged = plan

    def run_async(self) -> None:
        plan, self._staged = self._staged, None
        m, tp = self.model, self.tp
        T = plan.num_tokens
        fb = torch.from_numpy(plan.feedback_src).long()
        ids = torch.from_numpy(plan.host_ids).long().clone()
        use = fb >= 0
        ids[use] = self.sampled[fb[use]].long()
        x = self.ranks[0].embed[ids]
        pos = torch.from_numpy(plan.positions)
        kvh, hd = m.num_kv_heads // tp, m.head_dim
        for l in range(m.run_layers):
            o_sum = torch.zeros_like(x)
            h = ref.rmsnorm(x, self.ranks[0].layers[l % m.num_layers].ln_attn, m.rms_norm_eps)
            for r in range(tp):
                lw = self.ranks[r].layers[l % m.num_layers]
                qkv = h @ lw.wqkv.t()
                if lw.bqkv is not None:
                    qkv = qkv + lw.bqkv
                pool = self.kv_pool[r][l]
                q = ref.rope_append(qkv, pool, self.inv_freq, pos, plan.token_req, plan.kv_indptr,
                                    plan.kv_indices, q_heads=m.num_q_heads // tp, kv_heads=kvh, head_dim=hd,
                                    q_off=2 * kvh * hd, k_off=0, v_off=kvh * hd)
                att = ref.paged_attention(q, pool, plan.qo_indptr, plan.kv_indptr,
                                          torch.from_numpy(plan.kv_indices), plan.kv_last_page_len,
                                          q_heads=m.num_q_heads // tp)
                o_sum = o_sum + att @ lw.wo.t()
            x = x + o_sum
            h = ref.rmsnorm(x, self.ranks[0].layers[l % m.num_layers].ln_ffn, m.rms_norm_eps)
            d_sum = torch.zeros_like(x)
            for r in range(tp):
                lw = self.ranks[r].layers[l % m.num_layers]
                d_sum = d_sum + (torch.nn.functional.silu(h @ lw.wg.t()) * (h @ lw.wu.t())) @ lw.wd.t()
            x = x + d_sum
        rows = torch.from_numpy(plan.sample_rows).long()
        hs = ref.rmsnorm(x[rows], self.ranks[0].norm, m.rms_norm_eps)
        vl = self.ranks[0].lm_head.shape[0]
        logits = torch.cat([hs @ self.ranks[r].lm_head.t() for r in range(tp)], dim=1)[:, :m.vocab_size] \
            if tp * vl >= m.vocab_size else None
        self.last_logits = logits
        toks = logits.argmax(dim=-1).int()
        self.sampled[:toks.numel()] = toks
        self._inflight.append(toks.numpy().copy())

    def run_async_wait(self) -> np.ndarray:
        self._last = self._inflight.pop(0)
        return self._last

    def run(self, plan: BatchPlan) -> np.ndarray:
        self.update(plan)
        self.run_async()
        return self.run_async_wait()

    def getPipelineOutput(self) -> np.ndarray:
        return self._last

    @property
    def in_flight(self) -> int:
        return len(self._inflight)

    def check_status(self) -> None:
        pass

    def finalize(self) -> None:
        self._inflight.clear()
