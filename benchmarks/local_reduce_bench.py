#!/usr/bin/env python
"""The pairwise reduce recv[i] = op(recv[i], send[i]) on one GPU: this library's kernel against the ORIGINAL
library's own kernel on the same buffers.

The original's kernel (reference src/core/reduce.cu:9-100, dccl::do_device_reduce) is compiled unmodified by
baseline/build_reference_kernel.sh into baseline/_ref/libdccl_reference_reduce.so and called through its exported
C++ symbol; it is the only part of the original that builds without Derecho. Both sides run on the same device
buffers and the same stream, are timed with CUDA events after warm-up, and read 2 S and write S bytes of HBM per call
(S = count x element size), so bandwidth = 3 S / t against the measured copy rate of MEASURED_PEAKS.json.
Messages are larger than the 126 MB L2.

    python benchmarks/local_reduce_bench.py [--mb 256,1024] [--out results/local_reduce.json]
"""
import argparse
import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

REF_LIB = os.path.join(ROOT, "baseline", "_ref", "libdccl_reference_reduce.so")
REF_SYMBOL = "_ZN4dccl16do_device_reduceEPKvPvNS_14ncclDataType_tEmNS_11ncclRedOp_tEP11CUstream_st"
# name -> (enum value shared by both libraries, element size); the original has no bf16 kernel
TYPES = {"float32": (7, 4), "float16": (6, 2), "int32": (2, 4), "float64": (8, 8), "bfloat16": (9, 2)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", default="256,1024", help="message sizes in MB")
    ap.add_argument("--types", default="float32,float16,int32,bfloat16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    import torch
    from dccl_b200._lib import lib
    L = lib()
    ref = None
    if os.path.exists(REF_LIB):
        ref = getattr(ctypes.CDLL(REF_LIB), REF_SYMBOL)
        ref.restype = ctypes.c_int
        ref.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    peak = 6650.0
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:       # noqa: BLE001
        pass
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    rows = []
    for mb in [int(x) for x in args.mb.split(",")]:
        nbytes = mb << 20
        a = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        b = torch.ones(nbytes, dtype=torch.uint8, device="cuda")
        for name in args.types.split(","):
            dt, es = TYPES[name]
            count = nbytes // es

            def ours():
                rc = L.dccl_local_reduce_device(a.data_ptr(), b.data_ptr(), count, dt, 0, stream)
                assert rc == 0

            def theirs():
                rc = ref(b.data_ptr(), a.data_ptr(), dt, count, 0, stream)
                assert rc == 0, "the original's kernel returned %d" % rc

            def time_it(fn):
                a.zero_()
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) / args.iters

            ms = time_it(ours)
            row = {"dtype": name, "bytes": nbytes, "ours_ms": round(ms, 4), "ours_gbs": round(3 * nbytes / ms / 1e6, 1),
                   "ours_fraction_of_measured_copy_peak": round(3 * nbytes / ms / 1e6 / peak, 3)}
            if ref is not None and name != "bfloat16":
                rms = time_it(theirs)
                row.update({"reference_ms": round(rms, 4), "reference_gbs": round(3 * nbytes / rms / 1e6, 1), "speedup": round(rms / ms, 2)})
            else:
                row["reference_ms"] = None      # no bf16 kernel in the original; or the reference kernel is not built
            rows.append(row)
            print(json.dumps(row), flush=True)
        del a, b
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump({"peak_gbs": peak, "rows": rows}, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
