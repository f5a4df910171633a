"""Model / engine configuration.

One JSON file per (model, dense batch, pipeline type) with four sections, the schema of the
reference's ``pipeline/config_all/<model>/<batch>.json`` (e.g. llama2-70B/2048.json:1-60):

``model``            the Hugging Face ``config.json`` of the model, verbatim
``model_configs``    gpu_num, run_layer, allocate_kv_data_batch, frame_page_size, max_batch_size, ...
``pipeline_configs`` global_batch_size, nanobatch_1_size, kqv1_size, kqv3_size, gemm_op_tag[] (the
                     reference's CUTLASS tile tags: accepted and ignored) plus the sm_100a tuning
                     fields of this engine (``nanobatch_sizes``, ``sm_budget``, ``gemm_tile_n``, ...)
``serve_configs``    model id, actual_gpu_num, weight_path, hf_path, pipeline_type

The reference parses ``model`` + ``model_configs`` into a global struct and derives per-GPU sizes
(pipeline/include/config.h:90-111, pipeline/src/load_config.cu:11-112); :class:`ModelConfig` is that
struct, :class:`EngineConfig` holds the rest.
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Dict, List, Optional

PIPELINE_TYPES = (
    "PLLM", "NON_OVERLAP", "NANOBATCH", "PLLM_OFFLOAD", "LOCAL", "NON_OVERLAP_LOCAL",
    "NANOBATCH_LOCAL", "KQVBIAS", "NONOVERLAP_KQVBIAS", "NANOBATCH_KQVBIAS",
)


@dataclass
class ModelConfig:
    """Architecture + derived per-GPU sizes for tensor parallel degree ``tp``."""
    name: str = "llama"
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_q_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    qkv_bias: bool = False
    max_position_embeddings: int = 4096
    eos_token_id: int = 2
    bos_token_id: int = 1
    tp: int = 1                 # tensor-parallel degree the shapes are derived for ("vnranks")
    run_layers: int = 0         # layers executed (>= num_layers re-uses weights round-robin)

    def __post_init__(self):
        if self.run_layers <= 0:
            self.run_layers = self.num_layers
        if self.num_q_heads % self.tp or self.num_kv_heads % self.tp or self.intermediate_size % self.tp:
            raise ValueError(f"heads/ffn not divisible by tp={self.tp}")
        if self.num_q_heads % self.num_kv_heads:
            raise ValueError("q heads must be a multiple of kv heads")

    # ---- per-GPU sizes -------------------------------------------------------------------------
    @property
    def q_heads_local(self) -> int:
        return self.num_q_heads // self.tp

    @property
    def kv_heads_local(self) -> int:
        return self.num_kv_heads // self.tp

    @property
    def group_size(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    @property
    def q_size_local(self) -> int:
        return self.q_heads_local * self.head_dim

    @property
    def kv_size_local(self) -> int:
        return self.kv_heads_local * self.head_dim

    @property
    def qkv_size_local(self) -> int:
        """Columns of the packed K|V|Q projection on one GPU (``kqv_n`` in the reference)."""
        return self.q_size_local + 2 * self.kv_size_local

    @property
    def ffn_local(self) -> int:
        return self.intermediate_size // self.tp

    @property
    def vocab_local(self) -> int:
        """Rows of the vocab-sharded LM head per GPU, padded to a multiple of 8 columns."""
        per = (self.vocab_size + self.tp - 1) // self.tp
        return (per + 7) // 8 * 8

    def kv_bytes_per_token_local(self, dtype_bytes: int = 2) -> int:
        return 2 * self.kv_heads_local * self.head_dim * dtype_bytes * self.run_layers

    def param_count(self) -> int:
        h, f = self.hidden_size, self.intermediate_size
        per_layer = h * (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim + \
            self.num_q_heads * self.head_dim * h + 3 * h * f + 2 * h
        return per_layer * self.num_layers + 2 * self.vocab_size * h + h

    def matmul_flops_per_token(self) -> float:
        h, f = self.hidden_size, self.intermediate_size
        per_layer = h * (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim + \
            self.num_q_heads * self.head_dim * h + 3 * h * f
        return 2.0 * per_layer * self.run_layers

    @classmethod
    def from_hf(cls, hf: Dict[str, Any], *, tp: int = 1, run_layers: int = 0, name: str = "") -> "ModelConfig":
        heads = hf["num_attention_heads"]
        arch = (hf.get("architectures") or [""])[0]
        mtype = hf.get("model_type", "llama")
        return cls(
            name=name or mtype,
            hidden_size=hf["hidden_size"],
            intermediate_size=hf["intermediate_size"],
            num_layers=hf["num_hidden_layers"],
            num_q_heads=heads,
            num_kv_heads=hf.get("num_key_value_heads", heads),
            head_dim=hf.get("head_dim") or hf["hidden_size"] // heads,
            vocab_size=hf["vocab_size"],
            rms_norm_eps=hf.get("rms_norm_eps", 1e-5),
            rope_theta=float(hf.get("rope_theta", 10000.0)),
            rope_scaling=hf.get("rope_scaling"),
            qkv_bias=bool(hf.get("attention_bias", False)) or mtype == "qwen2" or "Qwen2" in arch,
            max_position_embeddings=hf.get("max_position_embeddings", 4096),
            eos_token_id=hf.get("eos_token_id", 2) if not isinstance(hf.get("eos_token_id"), list) else hf["eos_token_id"][0],
            bos_token_id=hf.get("bos_token_id", 1),
            tp=tp,
            run_layers=run_layers,
        )


@dataclass
class EngineConfig:
    """Everything that is not architecture: batching, nano-batches, SM budgets, serving options."""
    global_batch_size: int = 2048          # dense tokens per iteration
    nanobatch_sizes: List[int] = field(default_factory=list)   # token split of the dense batch
    page_size: int = 16
    num_pages: int = 0                     # KV pages per GPU; 0 = derive from free memory
    max_batch_size: int = 2048             # max concurrent requests in one iteration
    gpu_mem_fraction: float = 0.92
    pipeline_type: str = "PLLM"
    actual_gpu_num: int = 1
    gpu_num: int = 1
    # sm_100a tuning fields
    sm_budget: Dict[str, int] = field(default_factory=lambda: {"gemm": 0, "attn_decode": 0, "attn_prefill": 0, "comm": 0, "offload": 8})
    gemm_tile_n: Dict[str, int] = field(default_factory=dict)
    autotune_gemm: bool = True             # time candidate GEMM shapes at start-up and pin the fastest per op
    prefill_tc: bool = True                # head_dim 128: prefill attention on tcgen05 (else the mma.sync kernel)
    fuse_gemm_norm: bool = True            # one GPU: the RMSNorm after O / down comes out of the GEMM call
    prefill_beside_decode: bool = True     # prefill attention on a stream of its own, beside the decode kernel
    debug_guards: bool = False             # guard words around activation buffers, checked with the status word
    decode_tail_fraction: float = 0.0      # share of the decode context scheduled into the last nano-batch
    net_streams: int = 1                   # 2: collectives of odd nano-batches get a second network stream
    attn_overlap: bool = False             # TP: decode attention on its own stream under the other nano-batches' GEMMs
    cross_layer_pipeline: bool = False     # overlapped pipelines: the QKV / RoPE of layer l+1 of a nano-batch is issued
                                           # right behind its FFN of layer l, so its attention runs under the other
                                           # nano-batches' O / FFN GEMMs (software pipeline across layers)
    gate_gemm: bool = False                # TP: the GEMM behind an all-reduce + norm starts with the collective and waits
                                           # per 128-row block for the rows it reads (all-gather -> GEMM in one pipeline)
    o_allgather_nanos: List[int] = field(default_factory=list)   # TP: nano-batches whose O projection takes the
                                           # all-gather form (attention output gathered column-wise, N-split
                                           # weight, column blocks of the result gathered by the row owners)
                                           # instead of K-split weight + all-reduce
    prefill_impl: str = ""                 # "" = choose (ws for head_dim 128, mma otherwise or with prefill_tc off), "ws", "tc", "mma"
    decode_impl: str = ""                  # "" = per-warp cp.async rings, "tma" = TMA producer warp (head_dim 128)
    decode_stages: int = 0                 # decode attention pages in flight per warp: 0 = 3 (2 under attn_overlap), 2, 3
    gemm_shapes: Dict[str, Dict[str, int]] = field(default_factory=dict)   # "<op>.nb<k>" -> pinned launcher arguments
    decode_chunk_pages: int = 0            # 0 = choose per iteration
    use_cuda_graph: bool = False
    offload: bool = False
    fuse_gemm_rs: bool = False             # TP: K-split GEMMs push partial rows to their owners from the epilogue
    gemm_rs_staged: bool = False           # ... through shared memory and 256-byte bulk copies instead of 16-byte stores
    # serving
    model_id: str = ""
    weight_path: str = ""
    hf_path: str = ""
    gemm_op_tag: List[str] = field(default_factory=list)   # reference CUTLASS tags: kept, unused

    @property
    def overlap(self) -> bool:
        return self.pipeline_type in ("PLLM", "PLLM_OFFLOAD", "LOCAL", "KQVBIAS")

    @property
    def nanobatch(self) -> bool:
        return not self.pipeline_type.startswith("NON_OVERLAP") and not self.pipeline_type.startswith("NONOVERLAP")

    def resolved_nanobatches(self) -> List[int]:
        if not self.nanobatch:
            return [self.global_batch_size]
        if self.nanobatch_sizes:
            sizes = list(self.nanobatch_sizes)
            if sum(sizes) != self.global_batch_size:
                raise ValueError("nanobatch_sizes must sum to global_batch_size")
            return sizes
        return [self.global_batch_size]


@dataclass
class NanoflowConfig:
    model: ModelConfig
    engine: EngineConfig
    raw: Dict[str, Any] = field(default_factory=dict)

    def to_json(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)


def parse_config(raw: Dict[str, Any], *, tp: Optional[int] = None) -> NanoflowConfig:
    """Build the typed config from the four-section dictionary. Unknown keys are kept in ``raw``."""
    for sec in ("model", "model_configs", "pipeline_configs", "serve_configs"):
        if sec not in raw:
            raise ValueError(f"config is missing section '{sec}'")
    mc, pc, sc = raw["model_configs"], raw["pipeline_configs"], raw["serve_configs"]
    gpu_num = int(mc.get("gpu_num", 1))
    actual = int(sc.get("actual_gpu_num", gpu_num))
    model = ModelConfig.from_hf(raw["model"], tp=tp or gpu_num, run_layers=int(mc.get("run_layer", 0)),
                                name=sc.get("model", ""))
    ptype = sc.get("pipeline_type", "PLLM")
    if ptype not in PIPELINE_TYPES:
        raise ValueError(f"unknown pipeline_type '{ptype}' (known: {', '.join(PIPELINE_TYPES)})")
    gbs = int(pc.get("global_batch_size", mc.get("max_batch_size", 2048)))
    nano = pc.get("nanobatch_sizes")
    if nano is None and "nanobatch_1_size" in pc:
        n1 = int(pc["nanobatch_1_size"])
        nano = [n1, gbs - n1] if 0 < n1 < gbs else [gbs]
    page = int(mc.get("frame_page_size", 16))
    # Explicit "num_pages" wins; else the reference's rule allocate_kv_data_batch * 64 pages
    # (pipeline/src/vortexData.cu:10-31); 0 leaves the pool size to be derived from free memory.
    num_pages = int(mc.get("num_pages", 0)) or int(mc.get("allocate_kv_data_batch", 0)) * 64
    eng = EngineConfig(
        global_batch_size=gbs,
        nanobatch_sizes=list(nano or []),
        page_size=page,
        num_pages=num_pages,
        max_batch_size=int(mc.get("max_batch_size", 2048)),
        gpu_mem_fraction=float(mc.get("gpu_mem_fraction", 0.92)),
        pipeline_type=ptype,
        actual_gpu_num=actual,
        gpu_num=gpu_num,
        decode_chunk_pages=int(pc.get("decode_chunk_pages", 0)),
        use_cuda_graph=bool(pc.get("use_cuda_graph", False)),
        offload=ptype == "PLLM_OFFLOAD" or bool(pc.get("offload", False)),
        fuse_gemm_rs=bool(pc.get("fuse_gemm_rs", False)),
        gemm_rs_staged=bool(pc.get("gemm_rs_staged", False)),
        autotune_gemm=bool(pc.get("autotune_gemm", True)),
        prefill_tc=bool(pc.get("prefill_tc", True)),
        fuse_gemm_norm=bool(pc.get("fuse_gemm_norm", True)),
        prefill_beside_decode=bool(pc.get("prefill_beside_decode", True)),
        debug_guards=bool(pc.get("debug_guards", False)),
        decode_tail_fraction=float(pc.get("decode_tail_fraction", 0.0)),
        net_streams=int(pc.get("net_streams", 1)),
        attn_overlap=bool(pc.get("attn_overlap", False)),
        cross_layer_pipeline=bool(pc.get("cross_layer_pipeline", False)),
        prefill_impl=str(pc.get("prefill_impl", "")),
        gate_gemm=bool(pc.get("gate_gemm", False)),
        o_allgather_nanos=[int(k) for k in pc.get("o_allgather_nanos", [])],
        decode_impl=str(pc.get("decode_impl", "")),
        decode_stages=int(pc.get("decode_stages", 0)),
        model_id=sc.get("model", ""),
        weight_path=sc.get("weight_path", ""),
        hf_path=sc.get("hf_path", ""),
        gemm_op_tag=list(pc.get("gemm_op_tag", [])),
    )
    if "sm_budget" in pc:
        eng.sm_budget.update({k: int(v) for k, v in pc["sm_budget"].items()})
    if "gemm_tile_n" in pc:
        eng.gemm_tile_n.update({k: int(v) for k, v in pc["gemm_tile_n"].items()})
    if eng.nanobatch_sizes and sum(eng.nanobatch_sizes) != gbs:
        raise ValueError("nano-batch sizes must sum to global_batch_size")
    return NanoflowConfig(model=model, engine=eng, raw=raw)


def load_config(path, *, tp: Optional[int] = None) -> NanoflowConfig:
    with open(path) as f:
        raw = json.load(f)
    return parse_config(raw, tp=tp)


# --------------------------------------------------------------------------------------------------
# Built-in architectures (the models the reference ships configs for, plus the tiny test model)
# --------------------------------------------------------------------------------------------------
def _hf(hidden, ffn, layers, heads, kv, vocab, theta, *, mtype="llama", arch="LlamaForCausalLM", eps=1e-5,
        max_pos=4096, scaling=None, eos=2, bos=1, extra=None):
    d = {
        "architectures": [arch], "bos_token_id": bos, "eos_token_id": eos, "hidden_act": "silu",
        "hidden_size": hidden, "initializer_range": 0.02, "intermediate_size": ffn,
        "max_position_embeddings": max_pos, "model_type": mtype, "num_attention_heads": heads,
        "num_hidden_layers": layers, "num_key_value_heads": kv, "rms_norm_eps": eps,
        "rope_theta": theta, "rope_scaling": scaling, "tie_word_embeddings": False,
        "torch_dtype": "bfloat16", "vocab_size": vocab,
    }
    if extra:
        d.update(extra)
    return d


_LLAMA31_SCALING = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                    "original_max_position_embeddings": 8192, "rope_type": "llama3"}

MODEL_ARCHS: Dict[str, Dict[str, Any]] = {
    "tiny": _hf(256, 688, 2, 4, 2, 1024, 10000.0),
    # the same with 8 KV heads, so that it can be sharded over 8 ranks (head-parallel attention)
    "tiny8": _hf(1024, 2816, 2, 16, 8, 1024, 10000.0),
    "llama2-70B": _hf(8192, 28672, 80, 64, 8, 32000, 10000.0),
    "llama3-70B": _hf(8192, 28672, 80, 64, 8, 128256, 500000.0, max_pos=8192, eos=128001, bos=128000),
    "llama3.1-70B": _hf(8192, 28672, 80, 64, 8, 128256, 500000.0, max_pos=131072, scaling=_LLAMA31_SCALING,
                        eos=128001, bos=128000),
    "llama3-8B": _hf(4096, 14336, 32, 32, 8, 128256, 500000.0, max_pos=8192, eos=128001, bos=128000),
    "llama3.1-8B": _hf(4096, 14336, 32, 32, 8, 128256, 500000.0, max_pos=131072, scaling=_LLAMA31_SCALING,
                       eos=128001, bos=128000),
    "qwen2-72B": _hf(8192, 29568, 80, 64, 8, 152064, 1000000.0, mtype="qwen2", arch="Qwen2ForCausalLM",
                     eps=1e-6, max_pos=32768, eos=151643, bos=151643),
    "deepseek-67B": _hf(8192, 22016, 95, 64, 8, 102400, 10000.0, eps=1e-6, eos=100001, bos=100000),
    # Mixtral appears in the reference only as a JSON (no MoE code exists there); the dense
    # attention shapes are kept so the config parses, experts are not modelled.
    "mixtral-8-7B": _hf(4096, 14336, 32, 32, 8, 32000, 1000000.0, mtype="mixtral", arch="MixtralForCausalLM",
                        max_pos=32768, extra={"num_local_experts": 8, "num_experts_per_tok": 2}),
}

MODEL_IDS = {
    "llama2-70B": "meta-llama/Llama-2-70b-chat-hf", "llama3-70B": "meta-llama/Meta-Llama-3-70B-Instruct",
    "llama3.1-70B": "meta-llama/Meta-Llama-3.1-70B-Instruct", "llama3-8B": "meta-llama/Meta-Llama-3-8B-Instruct",
    "llama3.1-8B": "meta-llama/Meta-Llama-3.1-8B-Instruct", "qwen2-72B": "Qwen/Qwen2-72B-Instruct",
    "deepseek-67B": "deepseek-ai/deepseek-llm-67b-chat", "mixtral-8-7B": "mistralai/Mixtral-8x7B-Instruct-v0.1",
    "tiny": "nanoflow/tiny-llama-test", "tiny8": "nanoflow/tiny8-llama-test",
}


def default_nanobatches(gbs: int, pipeline_type: str) -> List[int]:
    if pipeline_type.startswith("NON_OVERLAP") or pipeline_type.startswith("NONOVERLAP"):
        return [gbs]
    # Two nano-batches in the reference's 5:11 proportion (640 / 1408 of 2048), rounded to whole
    # 128-row GEMM tiles so neither nano-batch ends in a ragged tile.
    n1 = max(128, int(round(gbs * 640 / 2048 / 128)) * 128)
    return [n1, gbs - n1] if gbs > n1 else [gbs]


def make_config(model: str, *, gpu_num: int = 1, global_batch_size: int = 2048,
                pipeline_type: Optional[str] = None, run_layer: int = 0, actual_gpu_num: Optional[int] = None,
                num_pages: int = 0, weight_path: str = "", **pipeline_overrides) -> Dict[str, Any]:
    """Generate the four-section dictionary for a built-in architecture."""
    if model not in MODEL_ARCHS:
        raise KeyError(f"unknown model '{model}' (known: {', '.join(MODEL_ARCHS)})")
    hf = copy.deepcopy(MODEL_ARCHS[model])
    if pipeline_type is None:
        if hf["model_type"] == "qwen2":
            pipeline_type = "KQVBIAS"
        else:
            pipeline_type = "PLLM" if gpu_num > 1 else "LOCAL"
    nano = default_nanobatches(global_batch_size, pipeline_type)
    raw = {
        "model": hf,
        "model_configs": {
            "gpu_num": gpu_num, "run_layer": run_layer or hf["num_hidden_layers"],
            "allocate_kv_data_batch": 0, "frame_page_size": 16, "max_batch_size": global_batch_size,
            "gpu_mem_fraction": 0.92,
        },
        "pipeline_configs": {
            "gemm_op_tag": [], "global_batch_size": global_batch_size,
            "nanobatch_1_size": nano[0], "nanobatch_sizes": nano,
            "kqv1_size": 0, "kqv3_size": 0,
            "sm_budget": {"gemm": 0, "attn_decode": 0, "attn_prefill": 0, "comm": 0, "offload": 8},
            "decode_chunk_pages": 0,
        },
        "serve_configs": {
            "model": MODEL_IDS.get(model, model), "actual_gpu_num": actual_gpu_num or gpu_num,
            "weight_path": weight_path or f"./nanoflow_weight_{model}/", "hf_path": "",
            "pipeline_type": pipeline_type,
        },
    }
    if num_pages:
        raw["model_configs"]["num_pages"] = num_pages
    raw["pipeline_configs"].update(pipeline_overrides)
    return raw


def builtin_config(model: str, **kw) -> NanoflowConfig:
    tp = kw.pop("tp", None)
    return parse_config(make_config(model, **kw), tp=tp)


CONFIG_DIR = Path(__file__).resolve().parent / "configs"


def shipped_config_path(model: str, variant: str = "2048") -> Path:
    return CONFIG_DIR / model / f"{variant}.json"


# --------------------------------------------------------------------------------------------------
# Shipped per-model configs: the variants the reference ships under pipeline/config_all/<model>/
# (768 / 1024 / 2048 dense batch, non-overlap, nanobatch-only, pllm-offload) plus a B200-sized one.
# --------------------------------------------------------------------------------------------------
def shipped_variants(model: str) -> Dict[str, Dict[str, Any]]:
    hf = MODEL_ARCHS[model]
    small = hf["hidden_size"] <= 4096
    gpus = 1 if small else 8
    local = "_LOCAL" if gpus == 1 else ""
    bias = hf["model_type"] == "qwen2"
    full = "KQVBIAS" if bias else ("LOCAL" if gpus == 1 else "PLLM")
    non = "NONOVERLAP_KQVBIAS" if bias else f"NON_OVERLAP{local}"
    nano = "NANOBATCH_KQVBIAS" if bias else f"NANOBATCH{local}"
    out = {}
    for gbs in (768, 1024, 2048):
        out[str(gbs)] = make_config(model, gpu_num=gpus, global_batch_size=gbs, pipeline_type=full)
    out["non-overlap"] = make_config(model, gpu_num=gpus, global_batch_size=2048, pipeline_type=non)
    out["nanobatch-only"] = make_config(model, gpu_num=gpus, global_batch_size=2048, pipeline_type=nano)
    if gpus > 1 and not bias:
        out["pllm-offload"] = make_config(model, gpu_num=gpus, global_batch_size=2048, pipeline_type="PLLM_OFFLOAD")
    # 180 GB of HBM3e per GPU holds a far larger KV pool than the 80 GB parts the 2048 batch was sized for
    big = 4096 if small else 8192
    out[f"b200-{big}"] = make_config(model, gpu_num=gpus, global_batch_size=big, pipeline_type=full,
                                     nanobatch_sizes=[big // 2, big // 2])
    # The reference's two scaled-down sets (pipeline/config_all/<model>/fewer_layers, correct_40G):
    # four layers' worth of weights with all layers run (weights re-used round-robin, so the timing is
    # that of the full model at a fraction of the memory), and a fixed small KV pool.
    for name in ("768", "1024", "2048", "non-overlap", "nanobatch-only"):
        few = copy.deepcopy(out[name])
        few["model_configs"]["run_layer"] = hf["num_hidden_layers"]
        few["model"]["num_hidden_layers"] = 4
        out[f"fewer_layers/{name}"] = few
    for name in ("1024" if small else "2048", "non-overlap", "nanobatch-only"):
        kv = copy.deepcopy(out[name])
        kv["model_configs"]["allocate_kv_data_batch"] = 100 if small else 400      # x 64 pages
        out[f"small_kv/{name}"] = kv
    return out


def write_shipped_configs(root: Optional[Path] = None) -> List[Path]:
    root = root or CONFIG_DIR
    written = []
    for model in MODEL_ARCHS:
        if model.startswith("tiny"):
            continue
        for name, raw in shipped_variants(model).items():
            path = root / model / f"{name}.json"
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps(raw, indent=2) + "\n")
            written.append(path)
    return written


if __name__ == "__main__":
    for p in write_shipped_configs():
        print(p)
