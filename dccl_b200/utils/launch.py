"""Start one process per rank on this machine and collect their results.

Used by tests, tools and the benchmark when no external launcher (torchrun) is
in charge. Ranks rendezvous on 127.0.0.1 through the DCCL_* variables.
"""
import os
import socket
import subprocess
import sys


def free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def spawn_ranks(argv, world, env_extra=None, per_rank_env=None, timeout=300, cwd=None, gpus=False, per_rank_argv=None):
    """Run ``argv`` (or ``per_rank_argv[rank]`` where given) once per rank; returns a list of CompletedProcess
    (stdout/stderr captured). A rank that outlives ``timeout`` is killed (only the processes started here)."""
    import tempfile
    port = free_port()
    procs, files = [], []
    for r in range(world):
        env = dict(os.environ)
        env.update({"DCCL_RANK": str(r), "DCCL_WORLD_SIZE": str(world), "DCCL_MASTER_ADDR": "127.0.0.1",
                    "DCCL_MASTER_PORT": str(port)})
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        if gpus:
            env["DCCL_LOCAL_DEVICE"] = str(r)
        if env_extra:
            env.update(env_extra)
        if per_rank_env and r in per_rank_env:
            env.update(per_rank_env[r])
        cmd = per_rank_argv[r] if per_rank_argv and r in per_rank_argv else argv
        # output goes to files, not pipes: a rank that prints a lot must never block (and with it the ranks that wait
        # for it in a collective) because nobody reads its pipe yet
        fo, fe = tempfile.TemporaryFile(mode="w+"), tempfile.TemporaryFile(mode="w+")
        files.append((fo, fe))
        procs.append(subprocess.Popen(cmd, env=env, cwd=cwd, stdout=fo, stderr=fe, stdin=subprocess.DEVNULL, text=True))
    import time
    deadline = time.monotonic() + timeout
    results = []
    for p, (fo, fe) in zip(procs, files):
        killed = False
        try:
            p.wait(timeout=max(0.0, deadline - time.monotonic()))
        except subprocess.TimeoutExpired:
            p.kill()
            p.wait()
            killed = True
        fo.seek(0)
        fe.seek(0)
        out, err = fo.read(), fe.read()
        fo.close()
        fe.close()
        if killed:
            err += "\n[killed after %d s]" % timeout
        results.append(subprocess.CompletedProcess(p.args, p.returncode, out, err))
    return results


def python_ranks(module_or_script, args, world, **kw):
    """spawn_ranks for a Python script / ``-m module``."""
    if module_or_script.endswith(".py"):
        argv = [sys.executable, module_or_script] + list(args)
    else:
        argv = [sys.executable, "-m", module_or_script] + list(args)
    return spawn_ranks(argv, world, **kw)


def main(argv=None):
    """``python -m dccl_b200.utils.launch -n 4 [--gpus] program [args...]``: one process per rank on this machine,
    output of every rank printed in rank order, exit code 0 only if every rank returned 0."""
    import argparse
    ap = argparse.ArgumentParser(prog="python -m dccl_b200.utils.launch")
    ap.add_argument("-n", "--ranks", type=int, default=2)
    ap.add_argument("--gpus", action="store_true", help="rank r drives GPU r (DCCL_LOCAL_DEVICE)")
    ap.add_argument("--timeout", type=int, default=600)
    ap.add_argument("program", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    prog = args.program[1:] if args.program[:1] == ["--"] else args.program
    if not prog:
        ap.error("no program given")
    if prog[0].endswith(".py"):
        prog = [sys.executable] + prog
    res = spawn_ranks(prog, args.ranks, timeout=args.timeout, gpus=args.gpus)
    worst = 0
    for r, p in enumerate(res):
        sys.stdout.write("".join("[%d] %s\n" % (r, ln) for ln in p.stdout.splitlines()))
        sys.stderr.write("".join("[%d] %s\n" % (r, ln) for ln in p.stderr.splitlines()))
        if p.returncode != 0:
            worst = p.returncode or 1
    return worst


if __name__ == "__main__":
    sys.exit(main())
