"""Module-level engine API with the function names of the reference's Python binding.

The reference exposes one process-wide pipeline through the module ``pllm_python``
(pipeline/src/pybind.cu:272-283: ``setModelConfig``, ``createModelWeight``, ``init``, ``config``,
``update``, ``run``, ``run_async``, ``run_async_wait``, ``getPipelineOutput``, ``finalize``, ``setRank``)
and feeds it structs of raw host pointers. Here the same call sequence drives an
:class:`nanoflow_b200.runtime.engine.Engine` (or the CPU backend when there is no GPU); the
per-iteration struct is the scheduler's :class:`~nanoflow_b200.serving.scheduler.BatchPlan`.

    import nanoflow_b200.pllm_python as pllm
    pllm.setModelConfig("nanoflow_b200/configs/llama3-8B/1024.json")
    weights = pllm.createModelWeight()            # random init; or nanoflow_b200.models.weights.load_rank_weights
    pllm.init(weights)
    pllm.config()                                  # builds the op graph, sizes the KV pool
    pllm.update(plan); pllm.run_async(); tokens = pllm.run_async_wait()
    pllm.finalize()
"""
from __future__ import annotations

import os
from typing import List, Optional

import numpy as np
import torch

from .config import NanoflowConfig, load_config, parse_config

_state = {"cfg": None, "weights": None, "engine": None, "rank": 0, "world": 1, "coll": None, "pages": None,
          "backend": None}


def _need(key: str, what: str):
    v = _state[key]
    if v is None:
        raise RuntimeError(f"{what} first")
    return v


def setRank(rank: int, world: int = 1) -> None:
    """This process's tensor-parallel rank (defaults come from RANK / WORLD_SIZE)."""
    _state["rank"], _state["world"] = int(rank), int(world)


def setModelConfig(config, *, backend: Optional[str] = None) -> NanoflowConfig:
    """``config``: path of a four-section JSON, the parsed dictionary, or a NanoflowConfig.
    ``backend``: "gpu", "cpu" or None (GPU when one is present)."""
    if _state["engine"] is not None:
        raise RuntimeError("finalize() the running pipeline before configuring another")
    world = int(os.environ.get("WORLD_SIZE", _state["world"]))
    _state["rank"] = int(os.environ.get("RANK", _state["rank"]))
    _state["world"] = world
    if isinstance(config, NanoflowConfig):
        cfg = config
    elif isinstance(config, dict):
        cfg = parse_config(config, tp=world if world > 1 else None)
    else:
        cfg = load_config(config, tp=world if world > 1 else None)
    _state["cfg"] = cfg
    _state["backend"] = backend or ("gpu" if torch.cuda.is_available() else "cpu")
    return cfg


def createModelWeight(seed: int = 0):
    """Random-init weights of the configured architecture: this rank's shard on the GPU backend, all
    ranks' shards (a list) on the CPU backend, which runs every rank in one process."""
    from .models import random_full_weights, random_rank_weights, shard_weights

    cfg = _need("cfg", "setModelConfig")
    m = cfg.model
    if _state["backend"] == "gpu":
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        return random_rank_weights(m, _state["rank"], m.tp, dev, seed=seed)
    fw = random_full_weights(m, seed=seed)
    return [shard_weights(fw, m, r, m.tp, dtype=torch.float32) for r in range(m.tp)]


def createInitData(num_pages: Optional[int] = None) -> dict:
    """KV pool size for ``init`` (the reference's init data also carries the weight and scratch
    pointers; here ``init`` takes the weights and the engine allocates its own buffers)."""
    return {"num_pages": num_pages}


def init(weights, init_data: Optional[dict] = None) -> None:
    _need("cfg", "setModelConfig")
    _state["weights"] = weights
    _state["pages"] = (init_data or {}).get("num_pages")


def config(config_data=None) -> None:
    """Build the pipeline (op graph, buffers, executor). ``config_data`` may override nano-batch sizes:
    ``{"nanobatch_sizes": [...]}``; GEMM tags of the reference's config data are accepted and unused."""
    cfg, weights = _need("cfg", "setModelConfig"), _need("weights", "init")
    if config_data and config_data.get("nanobatch_sizes"):
        cfg.engine.nanobatch_sizes = list(config_data["nanobatch_sizes"])
    if _state["backend"] == "gpu":
        from .runtime.engine import Engine

        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if _state["world"] > 1 and _state["coll"] is None:
            import torch.distributed as dist

            from .parallel.collectives import TpCollectives

            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=dev)
            _state["coll"] = TpCollectives(_state["rank"], _state["world"], dev)
        _state["engine"] = Engine(cfg, weights, device=dev, collectives=_state["coll"], num_pages=_state["pages"])
    else:
        from .runtime.cpu_backend import CpuEngine

        _state["engine"] = CpuEngine(cfg, weights, num_pages=_state["pages"] or 4096)


def num_pages() -> int:
    return int(_need("engine", "config").num_pages)


def update(plan) -> None:
    _need("engine", "config").update(plan)


def run(plan=None) -> np.ndarray:
    eng = _need("engine", "config")
    if plan is not None:
        eng.update(plan)
    eng.run_async()
    return eng.run_async_wait()


def run_async() -> None:
    _need("engine", "config").run_async()


def run_async_wait() -> np.ndarray:
    return _need("engine", "config").run_async_wait()


def getPipelineOutput() -> np.ndarray:
    """Tokens sampled by the last finished iteration, one per sampled request, int32."""
    return np.asarray(_need("engine", "config").getPipelineOutput(), dtype=np.int32)


def finalize() -> None:
    eng = _state["engine"]
    if eng is not None:
        eng.finalize()
    if _state["coll"] is not None:
        _state["coll"].close()
    _state.update(engine=None, weights=None, coll=None, pages=None)


def engine():
    """The engine object behind the module-level calls (None before ``config``)."""
    return _state["engine"]


__all__: List[str] = ["setRank", "setModelConfig", "createModelWeight", "createInitData", "init", "config", "update",
                      "run", "run_async", "run_async_wait", "getPipelineOutput", "finalize", "num_pages", "engine"]
