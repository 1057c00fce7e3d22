#!/usr/bin/env python
"""Turns the text output of build/dccl_sweep (benchmarks/run_sweep.sh) into a side-by-side table: for every
collective and size this library's time and bus bandwidth next to stock NCCL's, with the ratio.

    python benchmarks/sweep_table.py plain.log [sym.log] [ncclreg.log] > profiles/sweep_8gpu_bf16_vs_nccl.txt

The first log must hold the rows of both implementations on ordinary buffers (--impls dccl,nccl); further logs add
columns: rows of this library from a --symmetric run, rows of NCCL from a --nccl-register run. Rows are matched by
(collective, bytes). Times are microseconds per call (device time, maximum over ranks), bus bandwidth in GB/s by the
nccl-tests convention; ratio = NCCL time / this library's time on ordinary buffers.
"""
import sys


def parse(path):
    rows = {}
    for line in open(path):
        f = line.split()
        if len(f) < 7 or f[1] not in ("dccl", "nccl") or not f[2].isdigit():
            continue
        variant = " ".join(f[6:])
        rows[(f[0], f[1], variant.startswith("nccl-registered"), int(f[2]))] = (float(f[3]), float(f[5]), variant)
    return rows


def human(b):
    for unit, s in ((1 << 30, "GB"), (1 << 20, "MB"), (1 << 10, "KB")):
        if b >= unit:
            return ("%g %s" % (b / unit, s))
    return "%d B" % b


def main():
    if len(sys.argv) < 2:
        print(__doc__)
        return 1
    rows = {}
    for p in sys.argv[1:]:
        for k, v in parse(p).items():
            # a later log never replaces the ordinary-buffer rows of the first
            coll, impl, reg, b = k
            kind = "nccl_reg" if reg else impl if p == sys.argv[1] else ("sym" if impl == "dccl" else "nccl_reg")
            rows.setdefault((coll, b), {})[kind] = v
    colls = []
    for (coll, _b) in rows:
        if coll not in colls:
            colls.append(coll)
    for coll in colls:
        print("%s" % coll)
        print("%10s | %9s %8s %-22s | %9s %8s | %6s | %9s %8s %-10s | %9s %8s" %
              ("size", "ours us", "busBW", "variant", "NCCL us", "busBW", "ratio", "sym us", "busBW", "variant", "NCCLreg us", "busBW"))
        for (c, b) in sorted(k for k in rows if k[0] == coll):
            r = rows[(c, b)]
            o, n, s, g = r.get("dccl"), r.get("nccl"), r.get("sym"), r.get("nccl_reg")
            cell = lambda v, w=True: ("%9.1f %8.1f" % (v[0], v[1])) if v else ("%9s %8s" % ("-", "-"))     # noqa: E731
            ratio = "%6.2f" % (n[0] / o[0]) if o and n else "%6s" % "-"
            print("%10s | %s %-22s | %s | %s | %s %-10s | %s" %
                  (human(b), cell(o), o[2][:22] if o else "-", cell(n), ratio, cell(s), s[2][:10] if s else "-", cell(g)))
        print()
    return 0


if __name__ == "__main__":
    sys.exit(main())
