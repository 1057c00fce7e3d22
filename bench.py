#!/usr/bin/env python
"""Headline benchmark: all-reduce bus bandwidth (nccl-tests convention) on N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
           --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

One step = one ncclAllReduce (sum, bf16) of --bytes per rank through the library's public Python
API. The headline number ("value") is measured on ORDINARY device tensors (what a caller of NCCL
passes); "symmetric" is the same call on dcclMemAlloc memory, which the NVSwitch reduces in place.
The end-to-end number adds, in every step, the copy of that step's input from pinned host memory
and the read-back of the result. Times are CUDA-event times, maximum over ranks.
busBW = S/t * 2(n-1)/n; with one GPU the factor is undefined and the value is algBW = S/t of the
out-of-place local path. Every output element is compared with the exact sum (the inputs are
1/1024, so the sum is world/1024 in bf16 and fp32 alike); a wrong value ends the run with exit
code 3.

With more than one rank the same ranks then run the same measurement through stock NCCL
(torch.distributed): on ordinary tensors, and on tensors from NCCL's own registered allocator
(ncclMemAlloc + registration through torch's NCCL memory pool), the partner of "symmetric".
The line carries both under "nccl"; "vs_baseline" is value / NCCL's ordinary-tensor busBW from
the same run (the original library cannot be built here and publishes no numbers).

--impl nccl runs only the NCCL measurement, --impl reference reports that the original (a
C++/Derecho/RDMA library) cannot be installed here, --sweep adds a size sweep of all-reduce /
reduce-scatter / all-gather for every variant.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "allreduce_busbw"
UNAVAILABLE = ("the reference is a C++17/CMake library on top of Derecho, mutils, libfabric and spdlog; "
               "'pip install' of the reference tree fails (no setup.py / pyproject.toml) and its dependencies are not installable offline")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower() == "active" for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(self.samples)}


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def bus_factor(coll, n):
    if n <= 1:
        return 1.0
    return {"allreduce": 2.0 * (n - 1) / n, "reducescatter": (n - 1) / n, "allgather": (n - 1) / n}.get(coll, 1.0)


class Ours:
    name = "dccl_b200"

    def __init__(self, rank, world, local):
        import torch
        from dccl_b200 import Communicator
        self.torch = torch
        self.comm = Communicator(device=local)   # rank / world / rendezvous from the launcher's environment
        self.dev = torch.device("cuda", local)
        self.local = local
        self.world = world

    def alloc(self, numel, dtype, symmetric=True):
        if symmetric and self.world > 1:
            return self.comm.symmetric_empty(numel, dtype, self.local)
        return self.torch.empty(numel, dtype=dtype, device=self.dev)

    def free(self, t):
        if hasattr(t, "_dccl_ptr"):
            self.comm.free_symmetric(t)

    def all_reduce(self, s, r):
        self.comm.all_reduce(s, r, op="sum")
        return r

    def reduce_scatter(self, s, r):
        self.comm.reduce_scatter(s, r, op="sum")

    def all_gather(self, s, r):
        self.comm.all_gather(s, r)

    def set_algo(self, coll, algo):
        self.comm.set_algorithm(coll, algo)

    def launches(self):
        return self.comm.launches

    def host_max(self, x):
        import numpy as np
        a = np.array([x], dtype=np.float64)
        self.comm.all_reduce(a, op="max")
        return float(a[0])

    def barrier(self):
        import numpy as np
        a = np.zeros(1, dtype=np.int32)
        self.comm.all_reduce(a)

    def close(self):
        self.comm.finalize()


class StockNccl:
    name = "nccl"

    def __init__(self, rank, world, local):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
        self.dev = torch.device("cuda", local)
        self.world = world
        self._launch = 0
        self._pool = None

    def alloc(self, numel, dtype, symmetric=True):
        return self.torch.empty(numel, dtype=dtype, device=self.dev)

    def alloc_registered(self, numel, dtype):
        """A tensor from NCCL's own allocator (ncclMemAlloc), registered with the communicator: the buffers NCCL can
        hand to the switch without copies. Raises when this torch / NCCL cannot do it."""
        torch = self.torch
        backend = self.dist.group.WORLD._get_backend(self.dev)
        if self._pool is None:
            self._pool = torch.cuda.MemPool(backend.mem_allocator)
        with torch.cuda.use_mem_pool(self._pool):
            t = torch.empty(numel, dtype=dtype, device=self.dev)
        backend.register_mem_pool(self._pool)
        return t

    def free(self, t):
        pass

    def all_reduce(self, s, r):
        # torch's NCCL binding reduces in place: the input is restored (a device copy) by the caller outside the call
        self.dist.all_reduce(s)
        self._launch += 1
        return s

    def reduce_scatter(self, s, r):
        self.dist.reduce_scatter_tensor(r, s)
        self._launch += 1

    def all_gather(self, s, r):
        self.dist.all_gather_into_tensor(r, s)
        self._launch += 1

    def set_algo(self, coll, algo):
        pass

    def launches(self):
        return self._launch

    def host_max(self, x):
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def barrier(self):
        self.dist.barrier()

    def close(self):
        # tensors of the registered pool are gone by now; the pool must go before the communicator it is registered with
        if self._pool is not None:
            try:
                self.torch.cuda.synchronize()
                self.dist.group.WORLD._get_backend(self.dev).deregister_mem_pool(self._pool)
            except Exception:       # noqa: BLE001
                pass
            self._pool = None
            import gc
            gc.collect()
        self.dist.destroy_process_group()


def timed(backend, fn, steps, warmup):
    """ms per step: W warm-up calls, then K calls between two events, barrier + synchronize on both sides, max over ranks."""
    torch = backend.torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    backend.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    backend.barrier()
    torch.cuda.synchronize()
    return backend.host_max(e0.elapsed_time(e1) / steps)


def exact(t, world, torch):
    """Every element equals the exact sum of `world` inputs of 1/1024 (exact in bf16 and fp32 for world <= 256)."""
    return bool((t == world / 1024.0).all().item())


def measure(backend, args, numel, dtype, world, ours):
    """The three timed regions for one backend: ordinary tensors, registered / symmetric tensors, end to end."""
    torch = backend.torch
    nbytes = numel * (2 if dtype == torch.bfloat16 else 4)
    res = {"exact": True}
    factor = bus_factor("allreduce", world)

    def busbw(ms):
        return nbytes / (ms * 1e-3) / 1e9 * factor

    # ---- ordinary device tensors (the call as a user of NCCL makes it) ----
    src = backend.alloc(numel, dtype, symmetric=False)
    src.fill_(1.0 / 1024)
    dst = backend.alloc(numel, dtype, symmetric=False) if ours else src     # torch's NCCL binding reduces in place
    algo_seen = []

    def step():
        backend.all_reduce(src, dst)
        if ours and not algo_seen:
            algo_seen.append(backend.comm.last_algorithm("allreduce"))

    l0 = backend.launches()
    ms = timed(backend, step, args.steps, args.warmup)
    res["launches"] = (backend.launches() - l0) * args.steps // (args.steps + args.warmup)
    res["plain"] = {"ms_per_step": round(ms, 5), "busbw_gbs": round(busbw(ms), 3), "algbw_gbs": round(nbytes / (ms * 1e-3) / 1e9, 3)}
    res["algo"] = algo_seen[0] if algo_seen else "nccl"
    if ours:
        res["zero_copy"] = backend.comm.stat("zero_copy_calls") > 0
        ok = exact(dst, world, torch)
        res["plain"]["result_exact"] = ok
        res["exact"] = res["exact"] and ok

    # ---- buffers the library (or NCCL) allocated and registered itself ----
    res["registered"] = None
    if world > 1:
        try:
            if ours:
                ssrc = backend.alloc(numel, dtype, symmetric=True)
                sdst = backend.alloc(numel, dtype, symmetric=True)
            else:
                ssrc = backend.alloc_registered(numel, dtype)
                sdst = ssrc
            ssrc.fill_(1.0 / 1024)
            ms_r = timed(backend, lambda: backend.all_reduce(ssrc, sdst), args.steps, args.warmup)
            res["registered"] = {"ms_per_step": round(ms_r, 5), "busbw_gbs": round(busbw(ms_r), 3),
                                 "buffers": "dcclMemAlloc (symmetric, multicast-bound), out of place" if ours
                                            else "ncclMemAlloc through torch's NCCL memory pool, registered, in place"}
            if ours:
                res["registered"]["algorithm"] = backend.comm.last_algorithm("allreduce")
                ok = exact(sdst, world, torch)
                res["registered"]["result_exact"] = ok
                res["exact"] = res["exact"] and ok
                backend.free(ssrc)
                backend.free(sdst)
            del ssrc, sdst
        except Exception as e:      # noqa: BLE001  (an allocator this torch / NCCL does not have: say so, carry on)
            res["registered"] = {"unavailable": str(e)[:160]}

    # ---- end to end: pinned host input -> device -> all-reduce -> host, every step ----
    host_in = torch.empty(numel, dtype=dtype).pin_memory()
    host_in.fill_(1.0 / 1024)
    host_out = torch.empty(numel, dtype=dtype).pin_memory()

    def e2e_step():
        src.copy_(host_in, non_blocking=True)
        out = backend.all_reduce(src, dst)
        host_out.copy_(out, non_blocking=True)

    e2e_ms = timed(backend, e2e_step, args.e2e_steps, 3)
    ok = exact(host_out, world, torch)
    res["e2e"] = {"value": round(busbw(e2e_ms), 3), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": nbytes,
                  "d2h_bytes_per_step": nbytes, "steps": args.e2e_steps, "result_exact": ok}
    res["exact"] = res["exact"] and ok
    # ---- the same end-to-end step with the three legs overlapped (this library's host-buffer helper): a second figure,
    # never instead of the one above ----
    if ours:
        try:
            from dccl_b200.host_offload import HostAllReducer
            red = HostAllReducer(backend.comm, chunk_bytes=32 << 20, device=backend.local)
            pms = timed(backend, lambda: red(host_in, host_out, op="sum"), args.e2e_steps, 3)
            okp = exact(host_out, world, torch)
            red.close()
            res["e2e_pipelined"] = {"value": round(busbw(pms), 3), "unit": "GB/s", "ms_per_step": round(pms, 4), "h2d_bytes_per_step": nbytes,
                                    "d2h_bytes_per_step": nbytes, "steps": args.e2e_steps, "result_exact": okp,
                                    "how": "HostAllReducer: 32 MB chunks, host->device, switch and device->host on three streams"}
            # its own check stays in its own key: the figures above were checked on their own and stand without this extra
        except Exception as e:      # noqa: BLE001  (an extra; the measurement above stands without it)
            res["e2e_pipelined"] = {"unavailable": str(e)[:160]}
    del src, dst, host_in, host_out
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl", "reference"])
    ap.add_argument("--bytes", type=int, default=1 << 30, help="message bytes per rank for the headline all-reduce")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--no-nccl", action="store_true", help="skip the stock-NCCL measurement that follows this library's")
    ap.add_argument("--sweep", action="store_true", help="also sweep sizes and variants; table goes to --out")
    ap.add_argument("--out", default=os.path.join(ROOT, "results", "sweep.json"))
    ap.add_argument("--sweep-extra", action="store_true", help="broadcast / reduce / send-recv ring / dtype x operator rows")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--sweep-ctas", default="16,32,64,128")
    ap.add_argument("--sweep-min", type=int, default=1024, help="smallest message of the sweep")
    ap.add_argument("--sweep-unroll", default="4,8")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": UNAVAILABLE}))
        return 0

    import torch
    rank, world, local = env_rank_world()
    if world != args.gpus and rank == 0:
        print("note: --gpus %d but WORLD_SIZE is %d; using the launcher's value" % (args.gpus, world), file=sys.stderr)
    torch.cuda.set_device(local)
    ours = args.impl == "ours"
    backend = (Ours if ours else StockNccl)(rank, world, local)
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    es = 2 if args.dtype == "bf16" else 4
    numel = args.bytes // es
    nbytes = numel * es

    if args.algo != "auto":
        backend.set_algo("allreduce", args.algo)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    res = measure(backend, args, numel, dtype, world, ours)
    clocks = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary()

    sweep = None
    if args.sweep:
        sweep = run_sweep(backend, args, rank, world, dtype, es)
    if args.sweep_extra:
        sweep = (sweep or []) + run_extra(backend, args, rank, world)
    fabric = None
    if ours:
        try:    # the fabric as the communicator found it (NVLink links from NVML, -1 when that is not available)
            topo = backend.comm.topology()
            fabric = {"gpu": topo["gpus"][0]["name"], "multicast": bool(topo["gpus"][0]["multicast"]),
                      "nvlinks_active_min": min(g["nvlinks_active"] for g in topo["gpus"]),
                      "nvlinks_to_switch_min": min(g["nvlinks_to_switch"] for g in topo["gpus"]),
                      "all_pairs_peer_access": all(v in (1, 2, 255) for row in topo["peer_access"] for v in row)}
        except Exception as e:      # noqa: BLE001  (never let the report break the measurement)
            fabric = {"error": str(e)[:120]}
    backend.close()

    # ---- the comparator in the same run: the same ranks, the same bytes, steps and warm-up through stock NCCL ----
    nccl = None
    if ours and world > 1 and not args.no_nccl:
        try:
            nb = StockNccl(rank, world, local)
            nres = measure(nb, args, numel, dtype, world, False)
            nb.close()
            nccl = {"plain": nres["plain"], "registered": nres["registered"], "e2e": nres["e2e"]}
        except Exception as e:      # noqa: BLE001
            nccl = {"unavailable": str(e)[:200]}

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:       # noqa: BLE001
            pass
        link_gbs = 900.0
        ms = res["plain"]["ms_per_step"]
        value = res["plain"]["busbw_gbs"]
        roofline_ms = (2.0 * nbytes / (peaks.get("hbm_gbs", 6650.0) * 1e9) if world == 1
                       else 2.0 * nbytes * (world - 1) / world / (link_gbs * 1e9)) * 1e3
        vs = None
        if nccl and "plain" in nccl:
            vs = round(value / nccl["plain"]["busbw_gbs"], 4)
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": vs,
            "dtype": args.dtype, "data": "synthetic", "impl": backend.name,
            "config": {"model": "ncclAllReduce sum", "message_bytes_per_rank": nbytes, "global_batch": None, "seq_len": None,
                       "parallelism": "%d ranks, one per GPU" % world, "algorithm": res["algo"],
                       "buffers": "ordinary device tensors (torch.empty), out of place" if ours else "ordinary device tensors, in place",
                       "zero_copy": bool(res.get("zero_copy", False)),
                       "l2": "message (%d MiB) larger than the 126 MB L2" % (nbytes >> 20) if nbytes > (126 << 20) else "message fits L2: not flushed",
                       "value_is": "busBW = algBW*2(n-1)/n" if world > 1 else "algBW (one rank: out-of-place local path)",
                       "baseline": "stock NCCL 2.28 on ordinary tensors, same ranks and run (the original cannot be built offline and publishes no numbers)"},
            "algbw_gbs": res["plain"]["algbw_gbs"],
            "roofline": {"ms": round(roofline_ms, 5), "fraction": round(roofline_ms / ms, 4),
                         "of": "measured HBM copy" if world == 1 else "2S(n-1)/n over 900 GB/s per direction (P2P bound)"},
            "result_exact": bool(res["exact"]) if ours else None,
            "symmetric": res["registered"] if ours else None,
            "nccl": nccl if ours else {"registered": res["registered"]},
            "e2e": res["e2e"],
            "e2e_pipelined": res.get("e2e_pipelined"),
            "gpu_launches": int(res["launches"]) if ours else 0,
            "clocks": clocks,
        }
        if nccl and "plain" in nccl:
            line["ratios"] = {"plain_vs_nccl_plain": vs,
                              "symmetric_vs_nccl_registered": (round(res["registered"]["busbw_gbs"] / nccl["registered"]["busbw_gbs"], 4)
                                                               if res["registered"] and "busbw_gbs" in res["registered"] and nccl["registered"] and "busbw_gbs" in nccl["registered"] else None),
                              "symmetric_vs_nccl_plain": (round(res["registered"]["busbw_gbs"] / nccl["plain"]["busbw_gbs"], 4)
                                                          if res["registered"] and "busbw_gbs" in res["registered"] else None),
                              "e2e_vs_nccl_e2e": round(res["e2e"]["value"] / nccl["e2e"]["value"], 4)}
        if fabric is not None:
            line["fabric"] = fabric
        if sweep is not None:
            os.makedirs(os.path.dirname(args.out), exist_ok=True)
            with open(args.out, "w") as f:
                json.dump({"n_gpus": world, "impl": backend.name, "rows": sweep}, f, indent=1)
            line["sweep_file"] = os.path.relpath(args.out, ROOT)
        print(json.dumps(line))
    return 0 if (not ours or res["exact"]) else 3


def run_sweep(backend, args, rank, world, dtype, es):
    """busBW per (collective, variant, CTAs, unroll, size); sizes from 1 KB to the headline size.
    The pseudo-variant "nvls_sym" is the switch variant on symmetric (dcclMemAlloc) buffers."""
    rows = []
    sizes = []
    s = args.sweep_min
    while s <= args.bytes:
        sizes.append(s)
        s *= 8
    if sizes[-1] != args.bytes:
        sizes.append(args.bytes)
    ours = args.impl == "ours" and world > 1
    variants = {"allreduce": ["auto", "oneshot", "twoshot_ll", "twoshot", "ring", "rabenseifner", "nvls", "nvls_staged", "nvls_sym"],
                "reducescatter": ["auto", "twoshot", "ring", "nvls"], "allgather": ["auto", "twoshot", "ring", "nvls"]}
    if not ours:
        variants = {k: ["auto"] for k in variants}
    ctas_list = [int(x) for x in args.sweep_ctas.split(",")] if ours else [0]
    unroll_list = [int(x) for x in args.sweep_unroll.split(",")] if ours else [4]
    maxel = args.bytes // es
    src = backend.alloc(maxel, dtype, symmetric=False)
    dst = backend.alloc(maxel, dtype, symmetric=False)
    src.fill_(1.0 / 1024)
    ssrc = sdst = None
    if ours and backend.comm.has_multicast:
        ssrc = backend.alloc(maxel, dtype, symmetric=True)
        sdst = backend.alloc(maxel, dtype, symmetric=True)
        ssrc.fill_(1.0 / 1024)
    for coll, algos in variants.items():
        for algo in algos:
            if algo in ("nvls", "nvls_sym", "nvls_staged") and ours and not backend.comm.has_multicast:
                continue
            backend.set_algo(coll, "nvls" if algo in ("nvls_sym", "nvls_staged") else algo)
            if ours:
                backend.comm.set_param("pipe_min_mb", 0 if algo == "nvls_staged" else 16)
            a, b = (ssrc, sdst) if algo == "nvls_sym" else (src, dst)
            for size in sizes:
                if algo == "oneshot" and size > (128 << 10):
                    continue
                if algo == "twoshot_ll" and size > world * (512 << 10):
                    continue
                if algo in ("ring", "rabenseifner") and size > (256 << 20):
                    continue
                if algo == "nvls_staged" and size < (16 << 20):
                    continue
                for ctas in (ctas_list if (algo != "auto" and size >= (512 << 10)) else [0]):
                    for unroll in (unroll_list if algo in ("nvls", "nvls_sym", "nvls_staged") and size >= (512 << 10) else [4]):
                        if ours:
                            backend.comm.set_param("ctas", ctas)
                            backend.comm.set_param("unroll", unroll)
                        n_el = max(size // es, world * 8) // (world * 8) * (world * 8)
                        per = n_el // world
                        if coll == "allreduce":
                            fn = lambda: backend.all_reduce(a[:n_el], b[:n_el])   # noqa: E731
                            total = n_el * es
                        elif coll == "reducescatter":
                            fn = lambda: backend.reduce_scatter(a[:per * world], b[:per])   # noqa: E731
                            total = per * world * es
                        else:
                            fn = lambda: backend.all_gather(a[:per], b[:per * world])   # noqa: E731
                            total = per * world * es
                        steps = 200 if size <= (1 << 20) else 20 if size <= (64 << 20) else 8
                        ms = timed(backend, fn, steps, 5)
                        algbw = total / (ms * 1e-3) / 1e9
                        used = backend.comm.last_algorithm(coll) if args.impl == "ours" else "nccl"
                        rows.append({"coll": coll, "algo": algo, "ran": used, "ctas": ctas, "unroll": unroll, "bytes": total,
                                     "us": round(ms * 1e3, 3), "algbw_gbs": round(algbw, 3),
                                     "busbw_gbs": round(algbw * bus_factor(coll, world), 3)})
            backend.set_algo(coll, "auto")
    if ours:
        backend.comm.set_param("ctas", 0)
        backend.comm.set_param("unroll", 8)
    if ssrc is not None:
        backend.free(ssrc)
        backend.free(sdst)
    return rows


def run_extra(backend, args, rank, world, es_unused=None):
    """Rows for the other entry points: broadcast / reduce from both end ranks (fp32, 4 B - 256 MB), a ring of
    send/recv pairs (bf16, 64 MB), reduce-scatter / all-gather over dtypes and operators."""
    torch = backend.torch
    rows = []
    ours = args.impl == "ours"
    dev = backend.dev
    dist = getattr(backend, "dist", None)

    def record(coll, detail, nbytes, ms, factor=1.0):
        algbw = nbytes / (ms * 1e-3) / 1e9
        rows.append({"coll": coll, "detail": detail, "bytes": nbytes, "us": round(ms * 1e3, 3), "algbw_gbs": round(algbw, 3),
                     "busbw_gbs": round(algbw * factor, 3)})

    maxel = (256 << 20) // 4
    buf = torch.empty(maxel, dtype=torch.float32, device=dev)
    out = torch.empty(maxel, dtype=torch.float32, device=dev)
    buf.fill_(1.0)
    sizes = [4, 64, 1024, 16 << 10, 256 << 10, 4 << 20, 64 << 20, 256 << 20]
    for root in sorted({0, world - 1}):
        for size in sizes:
            n_el = max(1, size // 4)
            steps = 200 if size <= (1 << 20) else 20
            if ours:
                fb = lambda: backend.comm.broadcast(buf[:n_el], root=root)                    # noqa: E731
                fr = lambda: backend.comm.reduce(buf[:n_el], out[:n_el], op="sum", root=root)   # noqa: E731
            else:
                fb = lambda: dist.broadcast(buf[:n_el], src=root)       # noqa: E731
                fr = lambda: dist.reduce(out[:n_el], dst=root)          # noqa: E731
            record("broadcast", "root %d fp32" % root, n_el * 4, timed(backend, fb, steps, 5))
            record("reduce", "root %d fp32 sum" % root, n_el * 4, timed(backend, fr, steps, 5))
    # ring of send / recv pairs, 64 MB bf16: every rank sends to rank+1 and receives from rank-1
    if world > 1:
        n_el = (64 << 20) // 2
        sb = torch.ones(n_el, dtype=torch.bfloat16, device=dev)
        rb = torch.empty(n_el, dtype=torch.bfloat16, device=dev)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        if ours:
            from dccl_b200 import group_end, group_start

            def ring():
                group_start()
                backend.comm.send(sb, nxt)
                backend.comm.recv(rb, prv)
                group_end()
        else:
            def ring():
                ops = [dist.P2POp(dist.isend, sb, nxt), dist.P2POp(dist.irecv, rb, prv)]
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        record("sendrecv_ring", "64 MB bf16 per pair", n_el * 2, timed(backend, ring, 20, 5))
    # reduce-scatter / all-gather over dtypes and operators (per-rank counts 256 ... 16 M elements)
    tmap = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32, "int32": torch.int32}
    for tname, dt in tmap.items():
        esz = torch.empty((), dtype=dt).element_size()
        for per in [256, 64 << 10, 16 << 20]:
            src = torch.ones(per * world, dtype=dt, device=dev)
            dst = torch.empty(per * world, dtype=dt, device=dev)
            steps = 200 if per * esz <= (1 << 20) else 10
            for op in ["sum", "max", "min", "avg"]:
                if op == "avg" and not dt.is_floating_point and not ours:
                    continue
                if ours:
                    f = lambda: backend.comm.reduce_scatter(src, dst[:per], op=op)   # noqa: E731
                else:
                    rop = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.AVG}[op]
                    f = lambda: dist.reduce_scatter_tensor(dst[:per], src, op=rop)   # noqa: E731
                record("reducescatter", "%s %s" % (tname, op), per * world * esz, timed(backend, f, steps, 5), bus_factor("reducescatter", world))
            if ours:
                f = lambda: backend.comm.all_gather(src[:per], dst)   # noqa: E731
            else:
                f = lambda: dist.all_gather_into_tensor(dst, src[:per])   # noqa: E731
            record("allgather", tname, per * world * esz, timed(backend, f, steps, 5), bus_factor("allgather", world))
            del src, dst
    return rows


if __name__ == "__main__":
    sys.exit(main())
