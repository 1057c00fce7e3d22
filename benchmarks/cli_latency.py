#!/usr/bin/env python
"""Small-message latency through the C tools (no Python in the loop): runs dccl_cli and its stock-NCCL
twin nccl_cli on every visible GPU for a few sizes and prints their 'avg latency' lines as JSON.

    python benchmarks/cli_latency.py --gpus 8 --out results/cli_latency.json
"""
import argparse
import glob
import json
import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from dccl_b200.utils.launch import spawn_ranks  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--out", default=os.path.join(ROOT, "results", "cli_latency.json"))
    args = ap.parse_args()
    env = {}
    cands = glob.glob(os.path.join(sys.prefix, "lib", "python*", "site-packages", "nvidia", "nccl", "lib", "libnccl.so.2"))
    if cands:
        env["DCCL_NCCL_LIB"] = cands[0]
    rows = []
    for tool in ("dccl_cli", "nccl_cli"):
        for api in ("all_reduce", "reduce_scatter", "all_gather"):
            for count in (256, 16384, 262144):    # fp32 elements: 1 KB, 64 KB, 1 MB
                c = count if api == "all_reduce" else count * args.gpus
                argv = [os.path.join(ROOT, "build", tool), "-a", api, "-g", "auto", "-t", "float32", "-c", str(c), "-w", "50", "-r", "2000"]
                res = spawn_ranks(argv, args.gpus, env_extra=env, gpus=True, timeout=180, cwd="/tmp")
                m = re.search(r"avg latency: ([0-9.]+) us", res[0].stdout)
                rows.append({"tool": tool, "api": api, "bytes": c * 4, "us": float(m.group(1)) if m else None,
                             "rc": [p.returncode for p in res], "err": res[0].stderr[-300:] if not m else ""})
                print(rows[-1], flush=True)
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    json.dump({"n_gpus": args.gpus, "rows": rows}, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
