#!/usr/bin/env python
"""Short text summary of an Nsight Compute report: the figures the roofline reading needs, one per line.

Reads the report with `ncu -i <file> --page raw --csv` (works on a machine without a GPU) and prints, for every
captured launch (or the one chosen with --launch), duration, DRAM bytes and throughput, NVLink bytes where the
report has them, occupancy, the three largest warp stall reasons, registers and launch shape. The header lines
repeat the command that made the capture, so that the summary can be kept next to the code:

    python benchmarks/ncu_summary.py prof.ncu-rep --title "k_direct<bf16, sum>, 8 ranks emulated, 32 MB per rank" \\
        --command "ncu --set full --clock-control none -k regex:k_direct -c 1 -o prof python benchmarks/profile_emu.py ..." \\
        > profiles/ncu_direct.txt
"""
import argparse
import csv
import io
import os
import subprocess
import sys

WANTED = [
    "gpu__time_duration.sum",
    "dram__bytes_read.sum",
    "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "dram__cycles_active.avg",
    "lts__t_bytes.sum",
    "lts__throughput.avg.pct_of_peak_sustained_elapsed",
    "nvlrx__bytes.sum",
    "nvltx__bytes.sum",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "launch__registers_per_thread",
    "launch__grid_size",
    "launch__block_size",
    "launch__shared_mem_per_block_static",
    "launch__occupancy_limit_registers",
    "launch__occupancy_limit_shared_mem",
    "launch__waves_per_multiprocessor",
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"


def read_report(path, ncu="ncu"):
    p = subprocess.run([ncu, "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True)
    if p.returncode != 0:
        sys.exit("ncu could not read %s:\n%s" % (path, (p.stdout + p.stderr)[-2000:]))
    return parse_csv(p.stdout)


def parse_csv(text):
    """[(kernel name, {metric: (value, unit)})] from the raw page: a header row, a unit row, one row per launch."""
    start = text.find('"ID"')
    rows = list(csv.reader(io.StringIO(text[start:] if start >= 0 else text)))
    if len(rows) < 3:
        return []
    names, units = rows[0], rows[1]
    out = []
    for row in rows[2:]:
        if len(row) != len(names):
            continue
        rec = {names[i]: (row[i], units[i]) for i in range(len(names))}
        out.append((rec.get("Kernel Name", ("?", ""))[0], rec))
    return out


def summary_lines(rec):
    lines = []
    for m in WANTED:
        if m in rec and rec[m][0] != "":
            lines.append((m, rec[m][0], rec[m][1]))
    stalls = []
    for k, (v, u) in rec.items():
        if k.startswith(STALL_PREFIX) and k.endswith(STALL_SUFFIX) and "not_issued" not in k:
            try:
                stalls.append((float(v.replace(",", "")), k, u))
            except ValueError:
                pass
    for v, k, u in sorted(stalls, reverse=True)[:3]:
        lines.append((k, "%.3f" % v, u))
    return lines


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("report")
    ap.add_argument("--title", default="")
    ap.add_argument("--command", default="", help="the command line that made the capture (repeated in the header)")
    ap.add_argument("--launch", type=int, default=-1, help="index of the captured launch to print (default: all)")
    ap.add_argument("--ncu", default="ncu")
    args = ap.parse_args(argv)
    launches = read_report(args.report, args.ncu)
    if not launches:
        sys.exit("no launches in " + args.report)
    if args.title:
        print("# " + args.title)
    if args.command:
        print("# Plain run first (exit 0), then:")
        print("#   " + args.command)
    print("# Read with: ncu -i %s --page raw --csv (this file: python benchmarks/ncu_summary.py)" % os.path.basename(args.report))
    for i, (name, rec) in enumerate(launches):
        if args.launch >= 0 and i != args.launch:
            continue
        print()
        print("launch %d: %s" % (i, name))
        for m, v, u in summary_lines(rec):
            print("%-76s %s %s" % (m, v, u))
    return 0


if __name__ == "__main__":
    sys.exit(main())
