"""Worker script: many iterations through the host-only executor with several in flight, timed
iterations and graph mode mixed in. Run by tests/test_graph_cpu.py with a sanitizer's runtime
preloaded and the instrumented module's directory as the first argument."""
import sys

sys.path.insert(0, sys.argv[1])
import _executor_host as mod  # noqa: E402

ex = mod.Executor(0, 0, False, 2)
prev = -1
for i in range(40):
    deps = [prev] if prev >= 0 else []
    prev = ex.add_op(f"op{i}", mod.noop_fn(), bytes(16), i % 6, deps, [], [(0, i % 2, 4), (8, (i + 1) % 2, 8)])
ex.set_graph_mode(True)
tickets = []
for it in range(200):
    tickets.append(ex.submit([it, it + 1], it % 50 == 7))
    if len(tickets) >= 6:
        ex.wait(tickets.pop(0))
for t in tickets:
    ex.wait(t)
assert len(ex.timeline()) == 40
print("launches", ex.launches(), "graph launches", ex.graph_launches(), "rebuilds", ex.graph_rebuilds())
ex.close()
