"""The collective kernels on a machine without a GPU.

`make SIM=1 lib` compiles the kernel sources and the single-GPU emulation
harness as ordinary C++ against stand-in CUDA headers (csrc/sim/): every CUDA thread becomes an OS thread, flags are
host atomics, a packet is two 8-byte atomic halves. The tests of tests/test_gpu_emu.py then
run unchanged against build-sim/libdccl.so (DCCL_LIBRARY), which checks the flag protocol, the packet generations, the
staging geometry and the reductions of twoshot / oneshot / twoshot_ll / ring / rabenseifner / zero-copy two-shot /
send-recv, and (with a simulated multicast mapping) of the switch kernels. The scheduling of OS threads is far less regular than a GPU's, which is the point: an ordering the protocol
does not enforce shows up as a wrong result here (it did: the send/recv FIFO used to cut a short last chunk
differently from a full one, so that a sender could overwrite bytes another receiving CTA had not read yet).

A subset runs here (about a minute); the whole file passes as well:
    make SIM=1 lib && DCCL_LIBRARY=$PWD/build-sim/libdccl.so python -m pytest tests/test_gpu_emu.py -m gpu -q
(deselect the local-reduce and bounded-wait tests, whose kernels are not part of the simulation).
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(target_args, out):
    p = subprocess.run(["make", "-C", ROOT, "-j8", "lib"] + target_args, capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0 and os.path.exists(out), p.stdout[-2000:] + p.stderr[-2000:]
    return out


@pytest.fixture(scope="module")
def sim_lib():
    return build(["SIM=1"], os.path.join(ROOT, "build-sim", "libdccl.so"))


def test_emulation_tests_on_the_host_simulation(sim_lib):
    select = ("fp32_bf16_sizes or not_a_power_of_two or roots or send_recv_ring or ring_order or (two_shot_packet and 2) or guard_words or sequence_number "
              "or (all_to_all_as and (4-4 or 8-1)) or (zero_copy_broadcast and 3) or random_shapes")
    env = dict(os.environ, DCCL_LIBRARY=sim_lib)
    p = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_emu.py"), "-q", "-m", "gpu", "-p", "no:cacheprovider", "-k", select],
                       env=env, capture_output=True, text=True, timeout=1500)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-2000:]
    assert " passed" in p.stdout and "failed" not in p.stdout, p.stdout[-2000:]


def test_switch_kernels_on_the_host_simulation(sim_lib):
    """The multimem kernels with a simulated multicast mapping (a reserved address range that stands for the same
    offset in every rank's pool): staged forms of all five collectives, the pipelined all-reduce, the pipelined
    broadcast / reduce; world sizes 2, 3, 8, four dtypes, in place and unaligned, against the serial fold."""
    env = dict(os.environ, DCCL_LIBRARY=sim_lib)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "workers", "sim_switch_worker.py")], env=env, capture_output=True, text=True,
                       timeout=1500)
    assert p.returncode == 0 and "sim switch worker: ok" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


def test_range_checks_on_the_host_simulation():
    """The kernels compiled with their range checks (SIM=1 BOUNDS=1): normal runs pass with guard words on, and a run that
    is told a smaller staging area than its message needs is refused with the bounds code before it touches memory."""
    lib = build(["SIM=1", "BOUNDS=1"], os.path.join(ROOT, "build-sim-bounds", "libdccl.so"))
    env = dict(os.environ, DCCL_LIBRARY=lib)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "workers", "bounds_worker.py")], env=env, capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0 and "bounds worker: ok" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]


def test_thread_sanitizer_finds_no_unordered_access_between_ranks(tmp_path):
    """The simulation built with -fsanitize=thread: flags are atomics with the kernels' release / acquire order, data
    moves with plain loads and stores, so every access to staging, packets, FIFOs and user buffers that the protocol
    does not order is reported. The only reports allowed are on the simulation's stand-in for shared memory (one
    static per function instead of one per CTA)."""
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else None
    if cxx is None:
        pytest.skip("needs a system g++ with the sanitizer runtimes")
    flags = ["-std=c++17", "-O1", "-g", "-fsanitize=thread", "-fno-omit-frame-pointer", "-pthread", "-I" + os.path.join(ROOT, "include"),
             "-I" + os.path.join(ROOT, "csrc", "sim", "include"), "-DDCCL_HOST_SIM", "-DCACHELINE_SIZE=64", "-DENABLE_EVALUATION=1",
             "-fno-strict-aliasing", "-w"]
    srcs = ["csrc/core/config.cpp", "csrc/core/log.cpp", "csrc/api/names.cpp", "csrc/sim/sim_runtime.cpp", "csrc/gpu/emu.cu", "csrc/gpu/canary.cu",
            "csrc/kernels/twoshot.cu", "csrc/kernels/ring.cu", "csrc/kernels/hd.cu", "csrc/kernels/direct.cu", "csrc/kernels/oneshot_ll.cu",
            "csrc/kernels/ll_collectives.cu", "csrc/kernels/ll_twoshot.cu", "csrc/kernels/p2p.cu", "csrc/kernels/nvls.cu", "csrc/kernels/nvls_pipe.cu",
            "csrc/kernels/nvls_rooted.cu", "tests/sim/tsan_driver.cpp"]
    procs, objs = [], []
    for s in srcs:
        o = str(tmp_path / (os.path.basename(s) + ".o"))
        objs.append(o)
        procs.append(subprocess.Popen([cxx, "-x", "c++"] + flags + ["-c", os.path.join(ROOT, s), "-o", o], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=900)
        assert p.returncode == 0, out[-3000:]
    exe = str(tmp_path / "tsan_driver")
    p = subprocess.run([cxx] + [f for f in flags if f != "-w"] + objs + ["-o", exe, "-ldl", "-lrt"], capture_output=True, text=True, timeout=600)
    if p.returncode != 0 and "tsan" in (p.stdout + p.stderr).lower():
        pytest.skip("the sanitizer runtime is not installed")
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    run = subprocess.run([exe], cwd=str(tmp_path), capture_output=True, text=True, timeout=900, env=dict(os.environ, TSAN_OPTIONS="exitcode=0"))
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-3000:]
    assert "sendrecv rc=0" in run.stdout
    locations = [l.strip() for l in run.stderr.splitlines() if l.strip().startswith("Location is")]
    other = [l for l in locations if not ("::s_ok'" in l or "::s_fail'" in l or "::s_fine'" in l)]
    assert not other, "accesses that the protocol does not order:\n" + "\n".join(other[:10]) + "\n" + run.stderr[-4000:]
    assert run.stderr.count("WARNING: ThreadSanitizer") == len(locations), run.stderr[-4000:]
