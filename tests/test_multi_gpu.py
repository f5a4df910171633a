"""Multi-GPU tests (need >= 2 GPUs): collectives exactness, TP engine vs oracle, bounded peer waits.
Each case runs as child processes, one per GPU, NVLS off in NCCL (a rank leaving early must not
disturb multicast bindings)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _launch(case, n, port):
    # Heaps are plain CUDA IPC mappings unless the case is about the in-switch path, and NCCL keeps NVLS
    # off in every case that a rank may leave early.
    env = dict(os.environ, NANOFLOW_SYMM_BACKEND="ipc")
    if not case.endswith("_nvls"):
        env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_worker.py"), case]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    if res.returncode != 0 or f"MP_WORKER_OK {case}" not in res.stdout:
        fail = res.stdout[res.stdout.find("MP_WORKER_FAIL"):][:3000] if "MP_WORKER_FAIL" in res.stdout else ""
        raise AssertionError(fail + "\n--- stdout tail ---\n" + res.stdout[-1500:] + "\n--- stderr tail ---\n" + res.stderr[-1500:])
    return res.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("case,port", [("collectives", 29611), ("fused", 29614), ("engine", 29612), ("timeout", 29613),
                                       ("collectives_nvls", 29615), ("engine_nvls", 29616), ("engine_gate", 29617),
                                       ("engine_gate_nvls", 29618), ("engine_copy", 29619), ("engine_copy_nvls", 29620),
                                       ("engine_o1", 29630), ("engine_o1_nvls", 29631)])
def test_two_gpus(case, port):
    print(_launch(case, 2, port))


@pytest.mark.skipif(_ngpu() < 8, reason="needs 8 GPUs")
@pytest.mark.parametrize("case,port", [("collectives", 29621), ("fused", 29623), ("collectives_wide", 29624),
                                       ("engine", 29625), ("collectives_nvls", 29626), ("engine_nvls", 29627),
                                       ("engine_gate_nvls", 29628), ("engine_copy_nvls", 29629),
                                       ("engine_o1", 29632)])
def test_eight_gpus(case, port):
    print(_launch(case, 8, port))
