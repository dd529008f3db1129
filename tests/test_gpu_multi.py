"""Multi-GPU parity (one process per GPU, peer heap over CUDA IPC) against fixtures recorded from the
reference's own operators on CPU ranks. Skipped when the box has fewer GPUs than the case needs."""
import glob
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
_PORT = [29720]


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    _PORT[0] += 1
    try:
        mp.spawn(fn, args=(world, _PORT[0], *args, errq), nprocs=world, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")


def _world_of(path):
    with np.load(path) as f:
        return json.loads(str(f["spec"]))["world"]


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "usp_*.npz"))),
                         ids=lambda p: os.path.basename(p)[4:-4])
def test_usp_operator_matches_reference_fixture(path):
    from tests.multi_gpu_worker import usp_case
    _spawn(usp_case, _world_of(path), path)


@pytest.mark.parametrize("kind,world,ulysses", [("flux", 2, 2), ("sd3", 2, 2), ("flux", 2, 1), ("flux", 4, 2)])
def test_model_step_under_sequence_parallelism(kind, world, ulysses):
    """Whole tiny model, text stream sharded over the SP ranks and replicated, against the CPU oracle."""
    from tests.multi_gpu_worker import model_sp_case
    _spawn(model_sp_case, world, kind, ulysses)


@pytest.mark.parametrize("world", [2, 4])
def test_pipefusion_patch_ring(world):
    from tests.multi_gpu_worker import pipefusion_case
    _spawn(pipefusion_case, world)


@pytest.mark.parametrize("world", [2, 4])
def test_group_all_gather(world):
    from tests.multi_gpu_worker import all_gather_case
    _spawn(all_gather_case, world)


def test_barrier_timeout_is_reported_not_hung():
    from tests.multi_gpu_worker import barrier_timeout_case
    _spawn(barrier_timeout_case, 2)


def test_stage_handoff_to_decode_rank():
    from tests.multi_gpu_worker import handoff_case
    _spawn(handoff_case, 2)
