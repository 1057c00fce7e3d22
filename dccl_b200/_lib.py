"""Loader and ctypes prototypes of the native library (``libdccl.so``).

The library is built in-tree by ``make`` (``dccl_b200/lib/libdccl.so``). It is
loaded with ``ctypes``; nothing is compiled at import time. On a machine with a
GPU a missing library is an error, not a reason to fall back to something
slower.
"""
import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "lib", "libdccl.so")

_lib = None


def build(cuda=True, jobs=8, verbose=False):
    """Run ``make`` in the repository root (library + tools)."""
    cmd = ["make", "-C", _ROOT, "-j%d" % jobs, "CUDA=%d" % (1 if cuda else 0), "all"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        raise RuntimeError("building libdccl failed:\n" + (res.stdout or "")[-4000:] + (res.stderr or "")[-4000:])
    return LIB_PATH


def _declare(lib):
    c = ctypes
    vp, sz, i, cp = c.c_void_p, c.c_size_t, c.c_int, c.c_char_p
    sigs = {
        "dccl_comm_init": (i, [c.POINTER(vp)]),
        "dccl_get_unique_id": (i, [vp]),
        "dccl_comm_init_rank": (i, [c.POINTER(vp), i, vp, i]),
        "dccl_comm_finalize": (i, [vp]),
        "dccl_comm_abort": (i, [vp]),
        "dccl_topology_json": (i, [vp, cp, sz]),
        "dccl_debug_check": (i, [vp]),
        "dccl_barrier": (i, [vp]),
        "dccl_selftest_fd_exchange": (i, [vp]),
        "dccl_comm_shrink": (i, [vp, c.POINTER(vp)]),
        "dccl_world_size": (i, [vp]),
        "dccl_rank": (i, [vp]),
        "dccl_last_error": (i, [vp, c.POINTER(i), cp, sz]),
        "dccl_error_string": (cp, [i]),
        "dccl_comm_bind_device": (i, [vp, i]),
        "dccl_has_multicast": (i, [vp]),
        "dccl_launch_count": (c.c_ulonglong, [vp]),
        "dccl_cuda_device_count": (i, []),
        "dccl_comm_set_param": (i, [vp, cp, i]),
        "dccl_register": (i, [vp, vp, sz]),
        "dccl_deregister": (i, [vp, vp]),
        "dccl_mem_alloc": (i, [vp, c.POINTER(vp), sz]),
        "dccl_mem_free": (i, [vp, vp]),
        "dccl_all_reduce": (i, [vp, vp, sz, i, i, vp, vp]),
        "dccl_reduce_scatter": (i, [vp, vp, sz, i, i, vp, vp]),
        "dccl_all_gather": (i, [vp, vp, sz, i, vp, vp]),
        "dccl_broadcast": (i, [vp, vp, sz, i, i, vp, vp]),
        "dccl_reduce": (i, [vp, vp, sz, i, i, i, vp, vp]),
        "dccl_send": (i, [vp, sz, i, i, vp, vp]),
        "dccl_recv": (i, [vp, sz, i, i, vp, vp]),
        "dccl_all_to_all": (i, [vp, vp, sz, i, vp, vp]),
        "dccl_all_to_allv": (i, [vp, c.POINTER(sz), c.POINTER(sz), vp, c.POINTER(sz), c.POINTER(sz), i, vp, vp]),
        "dccl_gather": (i, [vp, vp, sz, i, i, vp, vp]),
        "dccl_scatter": (i, [vp, vp, sz, i, i, vp, vp]),
        "dccl_group_start": (i, []),
        "dccl_group_end": (i, []),
        "dccl_comm_stat": (c.c_ulonglong, [vp, cp]),
        "dccl_pool_bind": (None, [vp]),
        "dccl_is_symmetric": (i, [vp, vp, sz]),
        "dccl_selftest_board": (i, [vp, i]),
        "dccl_set_algorithm": (i, [vp, cp, cp]),
        "dccl_last_algorithm": (cp, [vp, cp]),
        "dccl_timestamp_log": (None, [c.c_ulonglong, c.c_ulonglong, c.c_ulonglong]),
        "dccl_timestamp_flush": (None, [cp, i]),
        "dccl_timestamp_clear": (None, []),
        "dccl_timestamp_size": (c.c_ulonglong, []),
        "dccl_config_reload": (None, []),
        "dccl_config_set": (None, [cp, cp]),
        "dccl_config_get": (i, [cp, cp, sz]),
        "dccl_config_parse_world": (i, [cp]),
        "dccl_slot_range": (None, [sz, c.c_uint, c.c_uint, sz, c.POINTER(sz), c.POINTER(sz)]),
        "dccl_reverse_bits": (c.c_uint, [c.c_uint, c.c_uint]),
        "dccl_log_two": (c.c_uint, [c.c_uint]),
        "dccl_size_of_type": (sz, [i]),
        "dccl_parse_type": (i, [cp]),
        "dccl_parse_op": (i, [cp]),
        "dccl_half_to_float": (c.c_float, [c.c_ushort]),
        "dccl_float_to_half": (c.c_ushort, [c.c_float]),
        "dccl_bf16_to_float": (c.c_float, [c.c_ushort]),
        "dccl_float_to_bf16": (c.c_ushort, [c.c_float]),
        "dccl_tuner_choose": (i, [cp, i, sz, i, cp, sz, c.POINTER(i)]),
        "dccl_tuner_choose_width": (i, [cp, i, sz, i, i, cp, sz, c.POINTER(i)]),
        "dccl_tuner_load_text": (i, [cp]),
        "dccl_tuner_dump": (sz, [cp, sz]),
    }
    cuda_only = {
        "dccl_emu_collective": (i, [cp, cp, i, i, i, sz, i, i, i, sz, i, sz, vp, vp]),
        "dccl_emu_sendrecv_ring": (i, [i, sz, i, i, i, vp, vp]),
        "dccl_emu_all_to_all": (i, [i, sz, i, i, vp, vp]),
        "dccl_emu_wait_probe": (i, [c.c_uint, c.POINTER(c.c_float)]),
        "dccl_nvml_link_report": (i, [cp, cp, sz]),
        "dccl_selftest_symmem": (i, [vp, i]),
        "dccl_emu_set_device_seq": (None, [i]),
        "dccl_emu_set_peer_buffers": (None, [i]),
        "dccl_emu_set_bcast_chunks": (None, [i]),
        "dccl_emu_switch_single": (i, [i, i, sz, i, i, vp, vp]),
        "dccl_local_reduce": (i, [vp, vp, sz, i, i]),
        "dccl_local_reduce_device": (i, [vp, vp, sz, i, i, vp]),
        "dccl_debug_bounds_build": (i, []),
        "dccl_selftest_canary": (i, []),
        "dccl_emu_set_guard": (None, [i]),
        "dccl_emu_set_mix": (i, [cp]),
        "dccl_emu_set_switch_form": (None, [i]),
        "dccl_emu_set_p2p_rendezvous": (None, [i]),
        "dccl_emu_set_pipe": (None, [sz, i]),
        "dccl_emu_declare_stage_bytes": (i, [sz]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for name, (res, args) in cuda_only.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
    return lib


def lib():
    """The loaded library (built on first use when the file is missing)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        # DCCL_LIBRARY: another build of the library, e.g. build-bounds/libdccl.so (make BOUNDS=1)
        path = os.environ.get("DCCL_LIBRARY") or LIB_PATH
        _lib = _declare(ctypes.CDLL(path))
    return _lib


def has_cuda_build():
    return hasattr(lib(), "dccl_emu_collective")
