"""Differentiable collectives (dccl_b200.ops) and the tensor / sequence parallel layers built on them, on CPU ranks:
every forward against the definition, every backward against the adjoint worked out by hand, a split MLP against
the unsplit one (outputs, input gradients, weight and bias gradients), and a pipeline of one stage per rank built
from the differentiable send / recv."""
import os

import pytest

from dccl_b200.utils.launch import python_ranks

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "workers", "tp_worker.py")


@pytest.mark.parametrize("world", [2, 3])
def test_differentiable_collectives_and_parallel_layers(dccl_lib, world):
    res = python_ranks(WORKER, [], world, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


@pytest.mark.parametrize("world", [1, 3])
def test_sharded_optimizer_matches_the_unsplit_one(dccl_lib, world):
    """dccl_b200.parallel.zero: reduce-scatter of the gradients, AdamW on this rank's slice, all-gather of the result,
    against plain AdamW on the mean loss; the optimizer state per rank shrinks with the world size."""
    res = python_ranks(os.path.join(HERE, "workers", "zero_worker.py"), [], world, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


@pytest.mark.parametrize("world", [1, 4])
def test_expert_parallel_layer_matches_all_experts_in_one_process(dccl_lib, world):
    """dccl_b200.parallel.expert_parallel: dispatch and combine through the differentiable all-to-all with per-peer
    counts; output, input gradient, expert gradients and the summed router gradient against the unsplit layer."""
    res = python_ranks(os.path.join(HERE, "workers", "moe_worker.py"), [], world, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


@pytest.mark.parametrize("world", [2, 3])
def test_ring_and_all_to_all_attention_match_attention_over_the_whole_sequence(dccl_lib, world):
    """dccl_b200.parallel.context_parallel: key / value blocks travelling the ring with a running softmax, and the
    sequence-to-heads all-to-all form; outputs and dq / dk / dv, with and without the causal mask."""
    res = python_ranks(os.path.join(HERE, "workers", "cp_worker.py"), [], world, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decoder_matches_the_unsplit_one(dccl_lib, world):
    """dccl_b200.models.llama_tp: heads and feed-forward columns dealt out over the ranks; loss, gradients of the
    replicated parameters and of every rank's slices against the unsplit decoder."""
    res = python_ranks(os.path.join(HERE, "workers", "llama_tp_worker.py"), [], world, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout


def test_layers_over_torch_distributed_adapter(dccl_lib):
    """The same worker with the collectives served by torch.distributed (gloo) through
    dccl_b200.parallel.torch_comm.TorchDistCommunicator: the layers do not depend on which library moves the data."""
    res = python_ranks(WORKER, ["--gloo"], 2, timeout=300)
    for r, p in enumerate(res):
        assert p.returncode == 0, "rank %d:\n%s\n%s" % (r, p.stdout[-3000:], p.stderr[-3000:])
        assert p.stdout.strip().splitlines()[-1].startswith("OK"), p.stdout
