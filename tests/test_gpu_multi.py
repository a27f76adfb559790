"""Multi-GPU tests (run only where at least two GPUs are visible): the decode
megakernel at cp = 2 (and 4 / 8 when present) over NVLink symmetric memory."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, worker="mp_layer_worker.py", token="MP_LAYER_OK", port=29500):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port + world), os.path.join(ROOT, "tests", worker)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and token in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
    print([l for l in r.stdout.splitlines() if token in l][-1])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decode_layer_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world)


@pytest.mark.parametrize("world", [2, 4])
def test_events_comm_scheduler_across_gpus(world):
    """Ping-pong / fan-in / fan-out hand-offs with a bulk-pushed payload checked behind flag-only waits,
    25 phases of a cross-rank task DAG, and the cross-GPU notify latency probe."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, "mp_events_worker.py", "MP_EVENTS_OK", port=29600)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_prefill_chunk_across_gpus(world):
    """Chunked prefill on the decode tiles at cp = world: per query token the causal selection and the
    merged attention against the oracle, on the owner rank; selections identical on all ranks."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, "mp_prefill_worker.py", "MP_PREFILL_OK", port=29700)
