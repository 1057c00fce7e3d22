"""Single-GPU run of the range-checking build of the library (make BOUNDS=1, loaded through DCCL_LIBRARY).

1. Every emulated variant still gives the right answer, with guard words on.
2. With the kernels told that a staging half has 32 KB (8 MB are allocated, so every address they could compute stays
   inside the allocation), a 256 KB message makes each staged variant refuse before its first access: the harness
   returns 100 + DEV_BOUNDS (3), and the same call passes again once the declaration is withdrawn.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from dccl_b200 import _lib  # noqa: E402
from dccl_b200.comm import DTYPE_NAMES, OPS  # noqa: E402
from dccl_b200.utils import oracle  # noqa: E402

DEV_BOUNDS = 3


def run(lib, kind, algo, n, count, ins):
    hin = np.concatenate(ins).astype(np.float32, copy=False)
    out_elems = count * n if kind == "allgather" else count
    hout = np.zeros(out_elems * n, dtype=np.float32)
    rc = lib.dccl_emu_collective(kind.encode(), algo.encode(), n, DTYPE_NAMES.index("float32"), OPS["sum"], count, 0, 3, 0, 0, 2,
                                 8 << 20, hin.ctypes.data, hout.ctypes.data)
    return rc, hout.reshape(n, out_elems)


def main():
    lib = _lib.lib()
    assert lib.dccl_debug_bounds_build() == 1, "DCCL_LIBRARY does not point at a range-checking build"
    n = 4
    lib.dccl_emu_set_guard(1)
    staged = [("allreduce", "twoshot"), ("allreduce", "ring"), ("allreduce", "rabenseifner"), ("reducescatter", "twoshot"),
              ("reducescatter", "ring"), ("allgather", "twoshot"), ("allgather", "ring"), ("broadcast", "twoshot"), ("reduce", "twoshot")]
    packets = [("allreduce", "oneshot"), ("allreduce", "twoshot_ll"), ("reducescatter", "oneshot"), ("allgather", "oneshot"),
               ("broadcast", "oneshot"), ("reduce", "oneshot"), ("reduce", "twoshot_ll")]
    for kind, algo in staged + packets:
        for count in [7, 8192]:
            in_count = count * n if kind == "reducescatter" else count
            ins = [oracle.make_input("float32", in_count, seed=100 + r) for r in range(n)]
            rc, out = run(lib, kind, algo, n, count, ins)
            assert rc == 0, (kind, algo, count, rc)
            if kind == "allreduce":
                assert np.allclose(out[0], oracle.fold(ins, "sum"), rtol=1e-5, atol=1e-5), (kind, algo, count)
    # told too little staging: refused, outputs untouched
    count = 65536
    for kind, algo in staged:
        in_count = count * n if kind == "reducescatter" else count
        ins = [oracle.make_input("float32", in_count, seed=200 + r) for r in range(n)]
        assert lib.dccl_emu_declare_stage_bytes(32 << 10) == 0
        rc, out = run(lib, kind, algo, n, count, ins)
        assert lib.dccl_emu_declare_stage_bytes(0) == 0
        assert rc == 100 + DEV_BOUNDS, (kind, algo, rc)
        assert not out.any(), (kind, algo, "output written although the call was refused")
        rc, out = run(lib, kind, algo, n, count, ins)
        assert rc == 0, (kind, algo, "after withdrawing the declaration", rc)
    print("bounds worker: ok")


if __name__ == "__main__":
    main()
