"""Single-GPU emulation tests of paths that have not run on hardware yet. Not collected by name: they are run in a child
process by tests/test_gpu_emu.py::test_paths_not_yet_run_on_hardware_in_a_child_process, and move into that file after
their first clean run."""
import numpy as np
import pytest

from dccl_b200.utils import oracle
from test_gpu_emu import close, emu, inputs_for, np_dtype

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [2, 4, 8])
def test_ring_kernel_adds_in_ring_order(dccl_lib, n):
    """fp32 sum through the ring kernel against a fold in the order the ring adds, shard by shard (shards are whole
    16-byte vectors): the bits must match."""
    for count in [1, 3, 257, 4096, 10007, 65536 + 5]:
        ins = inputs_for("float32", "sum", count, n, seed=count % 89)
        out = emu(dccl_lib, "allreduce", "ring", n, "float32", "sum", count, ins)
        assert np.array_equal(out[0], oracle.ring_fold_sum(ins, align=4)), (n, count)


@pytest.mark.parametrize("n", [2, 3, 8])
def test_two_shot_packet_all_reduce(dccl_lib, n):
    """Shards to their owners and folded shards to everybody, both as polled packets (no barrier); up to 256 KB per shard."""
    for name in ["float32", "bfloat16", "int8", "float64"]:
        for count in [1, 9, 4099, 65536 + 5, (n * (256 << 10)) // np.dtype(np_dtype(name)).itemsize]:
            for op in ["sum", "avg", "max"]:
                ins = inputs_for(name, op, count, n, seed=53)
                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                for in_place, misalign in [(0, 0), (1, 0), (0, 4)]:
                    out = emu(dccl_lib, "allreduce", "twoshot_ll", n, name, op, count, ins, in_place=in_place, misalign=misalign, iters=4, ctas=6)
                    for r in range(n):
                        assert close(out[r], want, name, n), (n, name, op, count, r, in_place, misalign)
                    for r in range(1, n):
                        assert np.array_equal(out[r], out[0]), (n, name, op, count, "ranks differ")
    # the same kernel as a reduce: folded shards go to the root only
    for root in {0, n - 1}:
        for count in [1, 5, 4099, 65536 + 5]:
            ins = inputs_for("float32", "sum", count, n, seed=59)
            for op in ["sum", "avg"]:
                out = emu(dccl_lib, "reduce", "twoshot_ll", n, "float32", op, count, ins, root=root, iters=4, ctas=6)
                assert close(out[root], oracle.fold(ins, op), "float32", n), ("reduce", n, root, count, op)
