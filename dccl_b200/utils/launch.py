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
    port = free_port()
    procs = []
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
        procs.append(subprocess.Popen(cmd, env=env, cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    results = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, err = p.communicate()
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
