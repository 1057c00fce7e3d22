"""Device collectives among real processes, one per GPU (needs at least two GPUs)."""
import os

import pytest

from conftest import gpu_count
from dccl_b200.utils.launch import python_ranks

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "workers", "gpu_worker.py")


def run(world, args, env=None, timeout=600):
    res = python_ranks(WORKER, args, world, env_extra=env, timeout=timeout, gpus=True)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout
    return res


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_every_variant_on_all_gpus():
    world = min(gpu_count(), 8)
    run(world, ["--suite", "basic"])


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_pipelined_switch_variant_on_small_and_odd_sizes():
    """The copy-in / switch / copy-out pipeline normally starts at 16 MB; here it serves everything above 256 KB."""
    world = min(gpu_count(), 8)
    run(world, ["--suite", "basic"], env={"DCCL_NVLS_PIPE_MIN_BYTES": str(256 << 10)})


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_unregistered_buffers_are_mapped_on_first_use_and_alignment_is_a_group_decision():
    """Large calls on ordinary tensors run zero-copy after an exchange of cudaIpc handles inside the call; freed and
    re-allocated buffers are mapped afresh; one rank with an unaligned pointer changes the path for all ranks alike."""
    run(min(gpu_count(), 8), ["--suite", "lazy"])


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_framework_memory_pool_hands_out_symmetric_memory_and_host_buffers_go_through_the_gpus():
    """torch.cuda.MemPool over the library's allocator hook: tensors made inside the pool are reduced in place by the
    switch; pinned host buffers are reduced by the chunked host -> device -> switch -> host helper."""
    world = min(gpu_count(), 4)
    res = python_ranks(os.path.join(HERE, "workers", "pool_worker.py"), [], world, timeout=600, gpus=True)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_messages_larger_than_staging_are_chunked():
    world = min(gpu_count(), 8)
    run(world, ["--suite", "chunk"], env={"DCCL_STAGING_BYTES": str(4 << 20)})


@pytest.mark.skipif(gpu_count() < 3, reason="needs three GPUs")
def test_every_variant_on_a_world_that_is_not_a_power_of_two():
    """Three ranks: halving and doubling with one leader / follower pair, next to the two-shot and ring forms."""
    run(3, ["--suite", "odd_world"])


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_peer_handles_fallback_without_multicast():
    """cudaIpc handles instead of cuMem descriptors: no multicast, peer loads / stores only."""
    run(2, ["--suite", "chunk"], env={"DCCL_POOL_MODE": "ipc", "DCCL_STAGING_BYTES": str(16 << 20)})


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_topology_packets_two_shot_and_composed_collectives():
    """dcclGetTopology, the two-shot packet all-reduce / reduce, all-to-all / gather / scatter on device buffers."""
    run(min(gpu_count(), 8), ["--suite", "extra"])


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_no_variant_writes_between_the_pool_regions():
    """The basic suite with guard words in the unused parts of every rank's pool, checked at the end."""
    run(min(gpu_count(), 8), ["--suite", "basic"], env={"DCCL_DEBUG_BOUNDS": "1"})


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
def test_pipelined_switch_broadcast_and_reduce():
    run(min(gpu_count(), 8), ["--suite", "rooted"])


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("worker", ["tp_worker.py", "zero_worker.py", "moe_worker.py", "cp_worker.py", "llama_tp_worker.py"])
def test_differentiable_collectives_and_parallel_layers_on_device_tensors(worker):
    """The workers of tests/test_ops.py with CUDA tensors: forward and adjoint collectives run as device kernels."""
    world = min(gpu_count(), 4)
    res = python_ranks(os.path.join(HERE, "workers", worker), ["--cuda"], world, timeout=600, gpus=True)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout
