#!/usr/bin/env python
"""Runs ONE collective kernel on one GPU with all ranks emulated (cooperative launch), sized for an
ncu capture: inputs larger than L2, a few GB on the device at most, two launches.

    python benchmarks/profile_emu.py --kind allreduce --algo twoshot --ranks 8 --mb 64 --ctas 16
    python benchmarks/profile_emu.py --kind allreduce --algo twoshot --peer-buffers --ranks 8 --mb 64   (zero-copy form, k_direct)
    python benchmarks/profile_emu.py --kind allreduce --algo rabenseifner --ranks 8 --mb 64               (k_hd)
    python benchmarks/profile_emu.py --kind reducescatter --algo oneshot --ranks 8 --mb 0.0625           (k_ll_collective)
    python benchmarks/profile_emu.py --kind sendrecv --ranks 8 --mb 64 --ctas 16                          (k_p2p, ring of pairs)
    python benchmarks/profile_emu.py --kind sendrecv --ranks 8 --mb 64 --ctas 16 --rendezvous             (k_p2p, direct stores into the receive buffers)
    python benchmarks/profile_emu.py --kind local_reduce --mb 256                                         (k_local_reduce, one rank)
    python benchmarks/profile_emu.py --kind switch --mb 256 --ctas 16     (k_nvls on a one-member multicast object, where the driver allows one)
    ncu --set full --clock-control none -k regex:k_twoshot -c 1 -o prof_twoshot \\
        python benchmarks/profile_emu.py --kind allreduce --algo twoshot --ranks 8 --mb 64 --ctas 16
"""
import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from dccl_b200._lib import lib  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="allreduce")
    ap.add_argument("--algo", default="twoshot")
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--mb", type=float, default=64.0, help="message MB per rank (fp32)")
    ap.add_argument("--ctas", type=int, default=16)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--peer-buffers", action="store_true", help="user buffers count as addressable by every rank (zero-copy two-shot)")
    ap.add_argument("--device-seq", action="store_true", help="sequence numbers counted on the device (the CUDA-graph mode)")
    ap.add_argument("--rendezvous", action="store_true", help="send / recv: large messages are stored straight into the receive buffers")
    args = ap.parse_args()
    L = lib()
    n = args.ranks
    L.dccl_emu_set_peer_buffers(1 if args.peer_buffers else 0)
    L.dccl_emu_set_device_seq(1 if args.device_seq else 0)
    if args.kind == "switch":
        count = int(args.mb * (1 << 20)) // 4
        hin = np.arange(count, dtype=np.float32)
        hout = np.zeros(count, dtype=np.float32)
        rc = L.dccl_emu_switch_single(7, 0, count, args.ctas, args.iters, hin.ctypes.data, hout.ctypes.data)
        print("rc", rc, "(-10: no multicast here, -11: set-up refused)", "match", bool(rc == 0 and np.array_equal(hin, hout)))
        sys.exit(0 if rc == 0 and np.array_equal(hin, hout) else 1)
    if args.kind == "local_reduce":
        count = int(args.mb * (1 << 20)) // 4
        a = np.ones(count, dtype=np.float32)
        b = np.full(count, 2.0, dtype=np.float32)
        rc = 0
        for _ in range(args.iters):
            rc = rc or L.dccl_local_reduce(a.ctypes.data, b.ctypes.data, count, 7, 0)
        print("rc", rc, "sample", a[:2])
        sys.exit(0 if rc == 0 else 1)
    if args.kind == "sendrecv":
        L.dccl_emu_set_p2p_rendezvous(1 if args.rendezvous else 0)
        nbytes = int(args.mb * (1 << 20))
        hin = np.ones(n * nbytes, dtype=np.uint8)
        hout = np.zeros(n * nbytes, dtype=np.uint8)
        rc = L.dccl_emu_sendrecv_ring(n, nbytes, 1, args.ctas, args.iters, hin.ctypes.data, hout.ctypes.data)
        print("rc", rc, "sample", hout[:2])
        sys.exit(0 if rc == 0 else 1)
    count = int(args.mb * (1 << 20)) // 4
    in_elems = count * n if args.kind == "reducescatter" else count
    out_elems = count * n if args.kind == "allgather" else count
    hin = np.ones(in_elems * n, dtype=np.float32)
    hout = np.zeros(out_elems * n, dtype=np.float32)
    # staging per half: the staged variants need up to (n + 1) / n of the message, Rabenseifner log2(n) + 1 areas of it
    stage = int(max(in_elems, out_elems) * 4 * (4.5 if args.algo == "rabenseifner" else 2.5)) + (1 << 20)
    rc = L.dccl_emu_collective(args.kind.encode(), args.algo.encode(), n, 7, 0, count, 0, args.ctas, 0, 0, args.iters, stage,
                               hin.ctypes.data, hout.ctypes.data)
    print("rc", rc, "sample", hout[:2])
    sys.exit(0 if rc == 0 else 1)


if __name__ == "__main__":
    main()
