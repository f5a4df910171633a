"""Tensor parallelism: symmetric heap over CUDA IPC, collective ops for the op graph."""
