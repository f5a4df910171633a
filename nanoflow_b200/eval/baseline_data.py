"""Published comparison numbers (tokens/s/GPU, Llama-2-70B, 8 x A100-80G, TP 8) as printed in the
reference's figures and plotting tables (figures/OfflineThroughput.png; pipeline/eval/baseline_data.py:3-92;
pipeline/eval/calculate_speedup.py:17). They are data for plots and speed-up tables, not measurements
of this engine.
"""

OFFLINE_FIXED = {   # workload -> system -> tokens/s/GPU
    "512-512": {"vLLM": 494, "DeepSpeed-FastGen": 490, "TensorRT-LLM": 735, "NanoFlow": 1286},
    "1024-512": {"vLLM": 552, "DeepSpeed-FastGen": 513, "TensorRT-LLM": 817, "NanoFlow": 1263},
    "512-1024": {"vLLM": 410, "DeepSpeed-FastGen": 372, "TensorRT-LLM": 636, "NanoFlow": 1212},
}
OFFLINE_REAL = {
    "splitwise": {"vLLM": 484, "DeepSpeed-FastGen": 548, "TensorRT-LLM": 831, "NanoFlow": 1259},
    "lmsys": {"vLLM": 251, "DeepSpeed-FastGen": 293, "TensorRT-LLM": 560, "NanoFlow": 1247},
    "sharegpt": {"vLLM": 255, "DeepSpeed-FastGen": 335, "TensorRT-LLM": 639, "NanoFlow": 1272},
}
OTHER_MODELS_1024_512 = {   # model -> (vLLM, NanoFlow, NanoFlow fraction of its own optimal)
    "llama3-70B": (593, 1306, 0.706), "qwen2-72B": (554, 1213, 0.674), "deepseek-67B": (532, 1147, 0.591),
    "mixtral-8-7B": (997, 6564, 0.637), "llama3-8B": (5187, 12756, 0.785),
}
OPTIMAL_LLAMA2_70B_A100 = 1857.0
HEADLINE = ("1024-512", 1263.0)


def speedup_table(ours_tok_s_per_gpu: float, workload: str = "1024-512"):
    row = OFFLINE_FIXED.get(workload) or OFFLINE_REAL[workload]
    return {name: ours_tok_s_per_gpu / v for name, v in row.items()}
