"""torch.distributed backend "dccl": every collective against values computed from the ranks' seeds,
DistributedDataParallel gradients against a serial reference. CPU tensors here; CUDA tensors in the
gpu-marked tests."""
import os

import pytest

from conftest import gpu_count
from dccl_b200.utils.launch import python_ranks

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "workers", "torch_worker.py")


def run(world, args, gpus=False, timeout=600):
    res = python_ranks(WORKER, args, world, timeout=timeout, gpus=gpus)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-2000:], p.stderr[-3000:])
        assert p.stdout.strip().endswith("OK")


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_and_ddp_on_cpu_tensors(world):
    run(world, ["--ddp", "--extra"])


@pytest.mark.gpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_collectives_and_ddp_on_cuda_tensors():
    run(min(gpu_count(), 8), ["--cuda", "--ddp"], gpus=True)


@pytest.mark.gpu
def test_single_gpu_process_group():
    run(1, ["--cuda", "--ddp"], gpus=True)


@pytest.mark.gpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_all_to_all_gather_scatter_batches_objects_subgroups_on_cuda_tensors():
    run(min(gpu_count(), 8), ["--cuda", "--extra"], gpus=True)
