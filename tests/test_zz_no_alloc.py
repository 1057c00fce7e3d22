"""The entry point that allocates nothing (csrc/kernels/noalloc_allreduce.h).

Some callers of the library may not allocate device memory when they need a reduction: all of it
may be handed out to a caching allocator or a KV-cache pool, or they sit on a path where the
device-wide synchronisation of cudaMalloc is not acceptable. For them the library exports
dccl_allreduce_one_device_noalloc, an all-reduce among buffers on one device whose scratch is a
fixed array inside the library image. This test calls it through its exported C symbol, the way
such a caller would, twice in a row on the same stream, and compares every rank's output with
what the allocating entry point (dccl_emu_collective, two-shot variant) returns for the same
inputs, and with a fold of the inputs computed on the CPU in fp64 / int64 (the two kernels share
their reduction code, so agreement between them alone would not show a fault in it). The buffers the TEST needs are made with torch; the entry point under test gets only
their addresses. The file sorts last so that a run that stops at the first failure has already
run everything else; it also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

from dccl_b200.comm import DTYPE_NAMES, OPS
from dccl_b200.utils import oracle

pytestmark = pytest.mark.gpu

MAX_BYTES = 256 * 1024


def _entry(lib):
    fn = lib.dccl_allreduce_one_device_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                   ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _reference(lib, n, name, op, count, ins):
    """Outputs of the existing (allocating) entry point: [n, count]."""
    np_dt = np.dtype(np.uint16) if name == "bfloat16" else np.dtype(name)
    hin = np.concatenate(ins).astype(np_dt, copy=False)
    hout = np.zeros(n * count, dtype=np_dt)
    rc = lib.dccl_emu_collective(b"allreduce", b"twoshot", n, DTYPE_NAMES.index(name), OPS[op], count, 0, 4, 0, 0, 1, 0,
                                 hin.ctypes.data, hout.ctypes.data)
    assert rc == 0
    return hout.reshape(n, count)


def _close(got, want, name, n):
    rtol, atol = oracle.tolerances(name, n)
    if rtol == 0.0:
        return np.array_equal(got, want)
    if name == "bfloat16":
        got, want = oracle.bf16_to_f32(got), oracle.bf16_to_f32(want)
    return np.allclose(got.astype(np.float64), want.astype(np.float64), rtol=rtol, atol=atol)


def _run(lib, torch, n, name, op, count, seed, in_place=False):
    fn = _entry(lib)
    np_dt = np.dtype(np.uint16) if name == "bfloat16" else np.dtype(name)
    ins = [oracle.make_input(name, count, seed=seed * 10 + r) for r in range(n)]
    want = _reference(lib, n, name, op, count, ins)
    # device buffers for the call under test (bit patterns travel as integers of the same width)
    carrier = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[np_dt.itemsize]
    d_in = [torch.from_numpy(x.view({1: np.uint8, 2: np.int16, 4: np.int32, 8: np.int64}[np_dt.itemsize]).copy()).to("cuda") for x in ins]
    d_out = d_in if in_place else [torch.full((count,), 0x55, dtype=carrier, device="cuda") for _ in range(n)]
    status = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    in_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in d_in])
    out_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in d_out])
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(n, DTYPE_NAMES.index(name), OPS[op], count, in_ptrs, out_ptrs, status.data_ptr(), stream)
    assert rc == 0, "entry point returned %d" % rc
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a wait inside the kernel gave up"
    serial = oracle.fold(ins, op, bf16=name == "bfloat16")      # independent of any kernel of the library
    for r in range(n):
        got = d_out[r].cpu().numpy().view(np_dt)
        assert _close(got, want[r], name, n), (n, name, op, count, r)
        assert _close(got, serial, name, n), ("against the serial fold", n, name, op, count, r)


def test_two_calls_in_a_row_match_the_allocating_entry_point(dccl_lib):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.cuda.set_device(0)
    # first call (this is also the per-device set-up), then a second one that reuses the same array with
    # another shape, so stale flags or staging bytes from the first call would show
    _run(dccl_lib, torch, 8, "float32", "sum", MAX_BYTES // 4, seed=1)
    _run(dccl_lib, torch, 3, "bfloat16", "avg", 10007, seed=2)
    # and more pairs: every width, in place, one rank, tiny messages
    _run(dccl_lib, torch, 4, "int32", "max", 4099, seed=3)
    _run(dccl_lib, torch, 4, "int32", "max", 4099, seed=4, in_place=True)
    _run(dccl_lib, torch, 2, "float64", "prod", 1000, seed=5)
    _run(dccl_lib, torch, 1, "float16", "sum", 5, seed=6)
    _run(dccl_lib, torch, 5, "uint8", "min", 3, seed=7)
    _run(dccl_lib, torch, 2, "float32", "sum", MAX_BYTES // 4, seed=8)   # the limit, worst case for staging


def test_requests_beyond_the_built_in_scratch_are_refused(dccl_lib, capfd):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    fn = _entry(dccl_lib)
    t = torch.zeros(16, dtype=torch.float32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(t.data_ptr(), t.data_ptr())
    assert fn(2, 7, 0, MAX_BYTES // 4 + 1, ptrs, ptrs, None, None) == -2     # too large: nothing is launched
    assert "above the limit" in capfd.readouterr().err
    assert fn(9, 7, 0, 4, ptrs, ptrs, None, None) == -1                        # more ranks than the array holds
    assert fn(2, 7, 0, 0, ptrs, ptrs, None, None) == 0                         # nothing to do
    torch.cuda.synchronize()
