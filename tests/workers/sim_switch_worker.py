"""The switch (multimem) kernels on the host simulation (DCCL_LIBRARY = build-sim/libdccl.so): staged forms of every
collective, the pipelined all-reduce and the pipelined broadcast / reduce, against the serial fold; then all-reduces that
follow two other collectives in the same world (sequences of different kernels share flags, packet generations and staging
halves). --all adds world size 2, one-element messages and more sequences."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from dccl_b200 import _lib  # noqa: E402
from dccl_b200.utils import oracle  # noqa: E402
from test_gpu_emu import close, emu, inputs_for  # noqa: E402


def main():
    L = _lib.lib()
    assert hasattr(L, "dccl_emu_set_switch_form"), "not the simulation build"
    cases = 0
    for form, kinds in ((0, ["allreduce", "reducescatter", "allgather", "broadcast", "reduce"]), (1, ["allreduce", "reducescatter"]), (2, ["broadcast", "reduce"])):
        L.dccl_emu_set_switch_form(form)
        for n in ((2, 3, 8) if "--all" in sys.argv[1:] else (3, 8)):
            for kind in kinds:
                for name, op in (("float32", "sum"), ("bfloat16", "avg"), ("int32", "max"), ("float16", "sum")):
                    if kind in ("allgather", "broadcast") and op != "sum":
                        continue
                    for count in ((1, 1031, 70001) if "--all" in sys.argv[1:] else (1031, 70001)):
                        for in_place, misalign in ((0, 0), (1, 0), (0, 4 if name in ("float32", "int32") else 2)):
                            root = n - 1
                            in_count = count * n if kind == "reducescatter" else count
                            ins = inputs_for(name, op, in_count, n, seed=71)
                            out = emu(L, kind, "nvls", n, name, op, count, ins, root=root, ctas=6, in_place=in_place, misalign=misalign,
                                      iters=3, stage=4 << 20)
                            bf = name == "bfloat16"
                            if kind == "allreduce":
                                want = oracle.fold(ins, op, bf16=bf)
                                ok = all(close(out[r], want, name, n) for r in range(n))
                            elif kind == "reduce":
                                ok = close(out[root], oracle.fold(ins, op, bf16=bf), name, n)
                            elif kind == "reducescatter":
                                want = oracle.fold(ins, op, bf16=bf)
                                ok = all(close(out[r], want[r * count:(r + 1) * count], name, n) for r in range(n))
                            elif kind == "allgather":
                                ok = all(np.array_equal(out[r], np.concatenate(ins)) for r in range(n))
                            else:
                                ok = all(np.array_equal(out[r], ins[root]) for r in range(n))
                            assert ok, (form, n, kind, name, op, count, in_place, misalign)
                            cases += 1
    # the pipelined forms with many chunks (4 KB each: up to 24 per call), other group sizes, in place and unaligned
    L.dccl_emu_set_switch_form(1)
    try:
        for chunk, nv, ctas in ((4096, 2, 7), (16384, 1, 12), (4096, 303, 9), (8192, 104, 11)):     # 303: three teams of one
            L.dccl_emu_set_pipe(chunk, nv)
            for n in (2, 5, 8):
                for kind in ("allreduce", "reducescatter"):
                    for name, op in (("float32", "sum"), ("bfloat16", "avg"), ("int64", "min")):
                        for count in (7, 4099, 50001):
                            for in_place, misalign in ((0, 0), (1, 0), (0, 8 if name == "int64" else 4 if name == "float32" else 2)):
                                ins = inputs_for(name, op, count * n if kind == "reducescatter" else count, n, seed=79)
                                out = emu(L, kind, "nvls", n, name, op, count, ins, ctas=ctas, in_place=in_place, misalign=misalign, iters=3, stage=4 << 20)
                                want = oracle.fold(ins, op, bf16=name == "bfloat16")
                                if kind == "allreduce":
                                    ok = all(close(out[r], want, name, n) for r in range(n))
                                else:
                                    ok = all(close(out[r], want[r * count:(r + 1) * count], name, n) for r in range(n))
                                assert ok, ("pipe", chunk, nv, ctas, n, kind, name, op, count, in_place, misalign)
                                cases += 1
        # a staging half much smaller than the message: the chunk slots are used as a ring (copy-in waits for the slot's
        # previous tenant to be gone) and chunk numbers run past one call's flag values into the following call numbers
        L.dccl_emu_set_pipe(4096, 2)
        for n in (2, 4, 8):
            for kind, counts in (("allreduce", (4099, 50001)), ("reducescatter", (4099,))):
                for name, op in (("float32", "sum"), ("bfloat16", "avg")):
                    for count in counts:
                        for in_place, misalign in ((0, 0), (1, 0), (0, 4 if name == "float32" else 2)):
                            ins = inputs_for(name, op, count * n if kind == "reducescatter" else count, n, seed=83)
                            out = emu(L, kind, "nvls", n, name, op, count, ins, ctas=7, in_place=in_place, misalign=misalign, iters=3, stage=64 << 10)
                            want = oracle.fold(ins, op, bf16=name == "bfloat16")
                            if kind == "allreduce":
                                ok = all(close(out[r], want, name, n) for r in range(n))
                            else:
                                ok = all(close(out[r], want[r * count:(r + 1) * count], name, n) for r in range(n))
                            assert ok, ("pipe ring", n, kind, name, op, count, in_place, misalign)
                            cases += 1
    finally:
        L.dccl_emu_set_pipe(16 << 20, 0)
    # zero-copy forms: the user buffers themselves are multicast-mapped (what dcclMemAlloc memory is)
    L.dccl_emu_set_switch_form(0)
    L.dccl_emu_set_peer_buffers(1)
    try:
        for n in (3, 8):
            for kind in ["allreduce", "reducescatter", "allgather", "broadcast", "reduce"]:
                for name, op in (("float32", "sum"), ("bfloat16", "avg"), ("int32", "min")):
                    if kind in ("allgather", "broadcast") and op != "sum":
                        continue
                    for count in (1024, 70000):
                        root = n - 1
                        in_count = count * n if kind == "reducescatter" else count
                        ins = inputs_for(name, op, in_count, n, seed=73)
                        out = emu(L, kind, "nvls", n, name, op, count, ins, root=root, ctas=4, iters=3, stage=4 << 20)
                        bf = name == "bfloat16"
                        if kind == "allreduce":
                            ok = all(close(out[r], oracle.fold(ins, op, bf16=bf), name, n) for r in range(n))
                        elif kind == "reduce":
                            ok = close(out[root], oracle.fold(ins, op, bf16=bf), name, n)
                        elif kind == "reducescatter":
                            want = oracle.fold(ins, op, bf16=bf)
                            ok = all(close(out[r], want[r * count:(r + 1) * count], name, n) for r in range(n))
                        elif kind == "allgather":
                            ok = all(np.array_equal(out[r], np.concatenate(ins)) for r in range(n))
                        else:
                            ok = all(np.array_equal(out[r], ins[root]) for r in range(n))
                        assert ok, ("zero-copy", n, kind, name, op, count)
                        cases += 1
    finally:
        L.dccl_emu_set_peer_buffers(0)
    # sequences: two other collectives before every call under test, in the same world and on the same buffers; what
    # they leave in flags, packet generations and staging halves is what the next kernel starts from
    import itertools
    pre = ["allreduce:oneshot", "broadcast:oneshot", "reduce:oneshot", "reducescatter:oneshot", "allreduce:twoshot_ll", "reduce:twoshot_ll",
           "allreduce:twoshot", "broadcast:twoshot", "allreduce:ring", "allreduce:nvls", "broadcast:nvls"]
    if "--all" not in sys.argv[1:]:
        pre = pre[:3] + pre[4:7] + pre[9:]
    n, count = 4, 1031
    try:
        for a, b in itertools.product(pre, pre):
            assert L.dccl_emu_set_mix((a + "," + b).encode()) == 2
            for algo in ["oneshot", "twoshot_ll", "twoshot", "nvls"]:
                ins = inputs_for("float32", "sum", count, n, seed=5)
                out = emu(L, "allreduce", algo, n, "float32", "sum", count, ins, root=1, iters=3)
                assert all(close(out[r], oracle.fold(ins, "sum"), "float32", n) for r in range(n)), ("after", a, b, algo)
                cases += 1
    finally:
        L.dccl_emu_set_mix(b"")
    print("sim switch worker: ok (%d cases)" % cases)


if __name__ == "__main__":
    main()
