#!/usr/bin/env python
"""Turn measured sweeps into a tuning table for DCCL_TUNE_FILE / [DCCL] tune_file.

Inputs are the JSON files written by `bench.py --sweep --out ...` (rows carry variant and CTA count) and by
`build/dccl_sweep --out ...` (one forced variant per file; give the CTA count of that run as FILE:CTAS).
For every collective and measured size the fastest (variant, CTAs) wins; neighbouring sizes with the same
winner are merged into one rule `<collective> <nranks> <max_bytes> <variant> <ctas>`. A size bucket reaches
from the previous measured size (exclusive) to its own (inclusive); the last one is open ended. Rows measured
on symmetric buffers go to the keys allreduce_sym / reducescatter_sym.

    python benchmarks/make_tune_table.py --in results/sweep.json --in results/sym_nvls16.json:16 --out tune.txt

`--builtin` writes the table that is compiled into the library instead (the starting point for a table of one's own; the
copy kept in cfg/tune_b200_nvswitch.txt is made this way and a unit test holds the two together):

    python benchmarks/make_tune_table.py --builtin --out cfg/tune_b200_nvswitch.txt
"""
import argparse
import json
import os
import sys

COLL = {"allreduce": "allreduce", "all_reduce": "allreduce", "reducescatter": "reducescatter", "reduce_scatter": "reducescatter",
        "allgather": "allgather", "all_gather": "allgather", "broadcast": "broadcast", "reduce": "reduce"}
REAL = {"oneshot", "twoshot", "twoshot_ll", "ring", "rabenseifner", "nvls"}


def load(spec, default_ctas):
    path, _, ctas = spec.partition(":")
    ctas = int(ctas) if ctas else default_ctas
    doc = json.load(open(path))
    n = int(doc.get("n_gpus", 0))
    file_sym = bool(doc.get("symmetric", False))
    out = []
    for r in doc.get("rows", []):
        if r.get("impl", "dccl") not in ("dccl", "ours"):
            continue
        coll = COLL.get(r.get("coll", ""))
        algo = r.get("algo", r.get("variant", ""))
        us = r.get("us")
        if coll is None or not us or us <= 0:
            continue
        sym = file_sym
        if algo == "nvls_sym":
            algo, sym = "nvls", True
        elif algo == "nvls_staged":
            continue            # a knob of the nvls variant, not a separate table entry
        ran = r.get("ran", algo)
        if algo not in REAL or ran != algo:
            continue            # "auto" rows, and forced variants that fell back to another one
        key = coll + "_sym" if sym and coll in ("allreduce", "reducescatter") else coll
        out.append((key, n, int(r["bytes"]), algo, int(r.get("ctas") or ctas), float(us)))
    return out


def build(rows):
    best = {}
    for key, n, nbytes, algo, ctas, us in rows:
        k = (key, n, nbytes)
        if k not in best or us < best[k][2]:
            best[k] = (algo, ctas, us)
    rules = []
    for key, n in sorted({(k[0], k[1]) for k in best}):
        sizes = sorted(k[2] for k in best if k[0] == key and k[1] == n)
        merged = []
        for s in sizes:
            algo, ctas, _ = best[(key, n, s)]
            if merged and merged[-1][1:] == (algo, ctas):
                merged[-1] = (s, algo, ctas)
            else:
                merged.append((s, algo, ctas))
        for i, (s, algo, ctas) in enumerate(merged):
            rules.append("%s %d %s %s %d" % (key, n, "inf" if i == len(merged) - 1 else str(s), algo, ctas))
    return rules


BUILTIN_HEADER = """# Variant table of dccl-b200 for B200 GPUs on one NVSwitch box: the table compiled into the library, in the format of
# DCCL_TUNE_FILE / [DCCL] tune_file. Written by: python benchmarks/make_tune_table.py --builtin
#
#   <collective> <nranks|*> <max_bytes> <algorithm> <ctas> [<element bytes>]
#
# Rules of one (collective, nranks) are tried in ascending max_bytes; an exact world size beats '*'. The rows come from
# sweeps of every variant and CTA count on 2, 4 and 8 B200s (bf16 and fp32 sum; 1 KB - 1 GB), best per size bucket.
# allreduce_sym / reducescatter_sym: buffers in symmetric memory (dcclMemAlloc). Where the row says twoshot and the peers
# can address the buffers (symmetric, registered, or mapped on first use from 4 MB on) the zero-copy peer form runs.
"""


def builtin_table():
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import ctypes
    from dccl_b200._lib import lib
    n = lib().dccl_tuner_dump(None, 0)
    buf = ctypes.create_string_buffer(n + 1)
    lib().dccl_tuner_dump(buf, n + 1)
    return buf.value.decode()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--in", dest="inputs", action="append", default=[], help="sweep JSON, optionally FILE:CTAS")
    ap.add_argument("--ctas", type=int, default=32, help="CTA count for rows that do not say")
    ap.add_argument("--builtin", action="store_true", help="write the table compiled into the library")
    ap.add_argument("--out", default="-")
    args = ap.parse_args()
    if args.builtin:
        text = BUILTIN_HEADER + builtin_table()
        if args.out == "-":
            sys.stdout.write(text)
        else:
            with open(args.out, "w") as f:
                f.write(text)
        return 0
    if not args.inputs:
        ap.error("give --in FILE (one or more) or --builtin")
    rows = []
    for spec in args.inputs:
        rows += load(spec, args.ctas)
    rules = build(rows)
    text = "# generated by benchmarks/make_tune_table.py from: %s\n" % " ".join(args.inputs) + "\n".join(rules) + "\n"
    if args.out == "-":
        sys.stdout.write(text)
    else:
        with open(args.out, "w") as f:
            f.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
