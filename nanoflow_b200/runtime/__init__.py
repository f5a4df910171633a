"""Per-GPU runtime: op graph, pipeline builder, executors, engine, CPU backend."""
