"""Weight conversion and loading in the reference's per-rank file format.

``save_weights`` writes ``weight_rank_{i}.pt``: a dict with the key set and tensor layout of the
reference converter (pipeline/utils/weightSaver.py:73-149): ``ModelNorm``, ``Embed`` ([vocab, hidden]),
``LmHead`` ([hidden, vocab], i.e. transposed) and per layer ``O1_l`` (o_proj split on N), ``O2_l``
(o_proj split on K), ``U_l`` / ``G_l`` (split on N), ``D_l`` (split on K), ``KQV_l`` (K | V | Q packed,
split on N), ``BKQV_l`` ([1, kqv_n], zeros when the model has no QKV bias), ``LNATT_l``, ``LNFFN_l``.
Every matrix is stored transposed to ``[K, N]`` row-major as the reference does, so files written by
either converter load here. The dtype is bf16 by default (the reference writes fp16).

``load_rank_weights`` turns one such file into :class:`RankWeights` in the ``[N, K]`` layout the sm_100a
kernels consume (a regenerable transpose, done once at load), the counterpart of
pipeline/utils/weightLoader.py:37-92 + ``modelWeightToGPU`` (pipeline/src/vortexData.cu:351-373).
The LM head is re-sharded along the vocabulary for tensor parallelism (the reference replicates it).
"""
from __future__ import annotations

import json
import os
import re
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig
from .llama import FullLayer, FullWeights, LayerWeights, RankWeights

HF_NAME_MAP = {
    "ln_attention": "model.layers.{i}.input_layernorm.weight",
    "w_d": "model.layers.{i}.mlp.down_proj.weight",
    "w_g": "model.layers.{i}.mlp.gate_proj.weight",
    "w_u": "model.layers.{i}.mlp.up_proj.weight",
    "ln_ffn": "model.layers.{i}.post_attention_layernorm.weight",
    "w_k": "model.layers.{i}.self_attn.k_proj.weight",
    "w_o": "model.layers.{i}.self_attn.o_proj.weight",
    "w_q": "model.layers.{i}.self_attn.q_proj.weight",
    "w_v": "model.layers.{i}.self_attn.v_proj.weight",
    "b_k": "model.layers.{i}.self_attn.k_proj.bias",
    "b_q": "model.layers.{i}.self_attn.q_proj.bias",
    "b_v": "model.layers.{i}.self_attn.v_proj.bias",
}


def full_weights_from_hf_state(state: Dict[str, torch.Tensor], num_layers: int) -> FullWeights:
    """Hugging Face ``state_dict`` names -> :class:`FullWeights` (no copies beyond what indexing makes)."""
    fw = FullWeights(embed=state["model.embed_tokens.weight"], norm=state["model.norm.weight"],
                     lm_head=state.get("lm_head.weight", state["model.embed_tokens.weight"]))
    for l in range(num_layers):
        g = lambda k: state[HF_NAME_MAP[k].format(i=l)]
        has_bias = HF_NAME_MAP["b_q"].format(i=l) in state
        fw.layers.append(FullLayer(wq=g("w_q"), wk=g("w_k"), wv=g("w_v"), wo=g("w_o"), wg=g("w_g"), wu=g("w_u"),
                                   wd=g("w_d"), ln_attn=g("ln_attention"), ln_ffn=g("ln_ffn"),
                                   bq=g("b_q") if has_bias else None, bk=g("b_k") if has_bias else None,
                                   bv=g("b_v") if has_bias else None))
    return fw


def load_hf_checkpoint(model_path: str) -> FullWeights:
    """Read every ``*.safetensors`` file of a Hugging Face snapshot directory."""
    from safetensors import safe_open  # optional dependency, only needed for real checkpoints

    with open(os.path.join(model_path, "config.json")) as f:
        num_layers = json.load(f)["num_hidden_layers"]
    state: Dict[str, torch.Tensor] = {}
    for fn in sorted(os.listdir(model_path)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_path, fn), "pt") as sf:
                for name in sf.keys():
                    state[name] = sf.get_tensor(name)
    return full_weights_from_hf_state(state, num_layers)


def _split(t: torch.Tensor, direction: str, n: int) -> List[torch.Tensor]:
    """'N' splits output rows, 'K' splits input columns, 'C' copies (weightSaver.py:22-40)."""
    if direction == "N":
        return list(t.split(t.shape[0] // n, 0))
    if direction == "K":
        return list(t.split(t.shape[1] // n, 1))
    return [t] * n


def rank_state_dicts(fw: FullWeights, nranks: int, dtype=torch.bfloat16) -> List[Dict[str, torch.Tensor]]:
    tr = lambda t: t.t().contiguous().to(dtype)           # stored [K, N] row-major
    out: List[Dict[str, torch.Tensor]] = [
        {"ModelNorm": fw.norm.to(dtype).clone(), "Embed": fw.embed.to(dtype).clone(), "LmHead": tr(fw.lm_head)}
        for _ in range(nranks)]
    for l, lay in enumerate(fw.layers):
        o1, o2 = _split(lay.wo, "N", nranks), _split(lay.wo, "K", nranks)
        u, g, d = _split(lay.wu, "N", nranks), _split(lay.wg, "N", nranks), _split(lay.wd, "K", nranks)
        k, q, v = _split(lay.wk, "N", nranks), _split(lay.wq, "N", nranks), _split(lay.wv, "N", nranks)
        if lay.bq is not None:
            bk, bq, bv = (list(b.split(b.shape[0] // nranks)) for b in (lay.bk, lay.bq, lay.bv))
        for r in range(nranks):
            kqv = torch.cat([tr(k[r]), tr(v[r]), tr(q[r])], dim=1)
            if lay.bq is not None:
                bkqv = torch.cat([bk[r], bv[r], bq[r]]).unsqueeze(0).to(dtype)
            else:
                bkqv = torch.zeros(1, kqv.shape[1], dtype=dtype)
            out[r].update({f"O1_{l}": tr(o1[r]), f"O2_{l}": tr(o2[r]), f"U_{l}": tr(u[r]), f"G_{l}": tr(g[r]),
                           f"D_{l}": tr(d[r]), f"KQV_{l}": kqv, f"BKQV_{l}": bkqv,
                           f"LNATT_{l}": lay.ln_attn.to(dtype).clone(), f"LNFFN_{l}": lay.ln_ffn.to(dtype).clone()})
    return out


def save_weights(fw: FullWeights, nranks: int, weight_dir: str, dtype=torch.bfloat16) -> List[str]:
    os.makedirs(weight_dir, exist_ok=True)
    paths = []
    for r, sd in enumerate(rank_state_dicts(fw, nranks, dtype)):
        p = os.path.join(weight_dir, f"weight_rank_{r}.pt")
        torch.save(sd, p)
        paths.append(p)
    return paths


def _num_layers(sd: Dict[str, torch.Tensor]) -> int:
    idx = [int(m.group(1)) for k in sd for m in [re.match(r"O1_(\d+)$", k)] if m]
    if not idx:
        raise ValueError("weight file holds no layer tensors (no O1_<l> keys)")
    return max(idx) + 1


def rank_weights_from_state(sd: Dict[str, torch.Tensor], cfg: ModelConfig, rank: int, tp: int,
                            device="cpu", dtype=torch.bfloat16, has_bias: Optional[bool] = None,
                            o1: bool = False) -> RankWeights:
    """One rank's file contents -> kernel layout ([N, K]; vocab-sharded LM head). ``o1`` also keeps the
    N-split O projection (``O1_<l>``) for pipelines that all-gather the attention output."""
    mv = lambda t: t.to(device=device, dtype=dtype).contiguous()
    L = _num_layers(sd)
    vl = cfg.vocab_local if cfg.tp == tp else ((cfg.vocab_size + tp - 1) // tp + 7) // 8 * 8
    head_full = sd["LmHead"].t()                                  # [vocab, hidden]
    head = torch.zeros(vl, head_full.shape[1], dtype=head_full.dtype)
    lo, hi = rank * vl, min(head_full.shape[0], (rank + 1) * vl)
    if hi > lo:
        head[:hi - lo] = head_full[lo:hi]
    layers = []
    for l in range(L):
        bias = sd.get(f"BKQV_{l}")
        use_bias = (cfg.qkv_bias if has_bias is None else has_bias) and bias is not None
        layers.append(LayerWeights(
            wqkv=mv(sd[f"KQV_{l}"].t()), wo=mv(sd[f"O2_{l}"].t()), wg=mv(sd[f"G_{l}"].t()), wu=mv(sd[f"U_{l}"].t()),
            wd=mv(sd[f"D_{l}"].t()), ln_attn=mv(sd[f"LNATT_{l}"]), ln_ffn=mv(sd[f"LNFFN_{l}"]),
            bqkv=mv(bias.reshape(-1)) if use_bias else None,
            wo1=mv(sd[f"O1_{l}"].t()) if (o1 and tp > 1) else None))
    return RankWeights(embed=mv(sd["Embed"]), norm=mv(sd["ModelNorm"]), lm_head=mv(head), layers=layers,
                       rank=rank, tp=tp)


def load_rank_weights(weight_dir: str, cfg: ModelConfig, rank: int, tp: int, device="cpu",
                      dtype=torch.bfloat16, o1: bool = False) -> RankWeights:
    path = os.path.join(weight_dir, f"weight_rank_{rank}.pt")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} not found: run save_weights first (or use random weights)")
    sd = torch.load(path, map_location="cpu")
    return rank_weights_from_state(sd, cfg, rank, tp, device=device, dtype=dtype, o1=o1)


def load_weights(nranks: int, weight_dir: str, cfg: ModelConfig, device="cpu", dtype=torch.bfloat16):
    """All ranks' shards, loaded in a thread pool like the reference loader."""
    with ThreadPoolExecutor(max_workers=min(8, nranks)) as ex:
        return list(ex.map(lambda r: load_rank_weights(weight_dir, cfg, r, nranks, device, dtype), range(nranks)))


def convert_hf_checkpoint(hf_path: str, weight_dir: str, nranks: int, dtype=torch.bfloat16) -> List[str]:
    """Hugging Face snapshot directory -> ``weight_rank_<i>.pt`` files for ``nranks`` ranks."""
    os.makedirs(weight_dir, exist_ok=True)
    return save_weights(load_hf_checkpoint(hf_path), nranks, weight_dir, dtype=dtype)


def ensure_converted(weight_dir: str, hf_path: str, nranks: int, dtype=torch.bfloat16) -> bool:
    """Convert once: if ``weight_dir`` lacks the per-rank files and ``hf_path`` is a local snapshot with
    safetensors files, write them (the reference's serving script does the same when its weight path is
    missing, pipeline/utils/serve_8B.py:613-623). Returns whether the per-rank files exist afterwards."""
    have = weight_dir and all(os.path.exists(os.path.join(weight_dir, f"weight_rank_{r}.pt")) for r in range(nranks))
    if have:
        return True
    if not (weight_dir and hf_path and os.path.isdir(hf_path) and
            any(fn.endswith(".safetensors") for fn in os.listdir(hf_path))):
        return False
    convert_hf_checkpoint(hf_path, weight_dir, nranks, dtype)
    return True


def main(argv=None) -> int:
    """``python -m nanoflow_b200.models.weights --hf <snapshot dir> --out <dir> --nranks 8``"""
    import argparse

    ap = argparse.ArgumentParser(description="Hugging Face safetensors -> per-rank weight files "
                                             "(the reference's weightSaver.py layout)")
    ap.add_argument("--hf", required=True, help="local snapshot directory (config.json + *.safetensors)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--nranks", type=int, default=8)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    a = ap.parse_args(argv)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    for path in convert_hf_checkpoint(a.hf, a.out, a.nranks, dt):
        print(path)
    return 0


if __name__ == "__main__":
    import sys

    sys.exit(main())
