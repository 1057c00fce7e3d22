"""Python face of the communicator: a thin object over the C API.

Buffers are passed as raw addresses, so the same calls serve numpy arrays
(host collectives over shared memory) and torch CUDA tensors (device kernels).
Counterpart of the C++ API in ``include/dccl/dccl.hpp`` (which follows
reference include/dccl/dccl.hpp:143-474).
"""
import ctypes
import os

import numpy as np

from ._lib import lib

# ncclDataType_t / ncclRedOp_t values
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(10)
SUM, PROD, MAX, MIN, AVG = range(5)
OPS = {"sum": SUM, "prod": PROD, "max": MAX, "min": MIN, "avg": AVG}
DTYPE_NAMES = ["int8", "uint8", "int32", "uint32", "int64", "uint64", "float16", "float32", "float64", "bfloat16"]
DTYPE_SIZES = [1, 1, 4, 4, 8, 8, 2, 4, 8, 2]

_NP_TO_DCCL = {
    np.dtype(np.int8): INT8, np.dtype(np.uint8): UINT8, np.dtype(np.int32): INT32, np.dtype(np.uint32): UINT32,
    np.dtype(np.int64): INT64, np.dtype(np.uint64): UINT64, np.dtype(np.float16): FLOAT16,
    np.dtype(np.float32): FLOAT32, np.dtype(np.float64): FLOAT64,
}


class DcclError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        msg = lib().dccl_error_string(code).decode()
        super().__init__("%s failed: %s (ncclResult_t %d)" % (what, msg, code))


def _check(code, what):
    if code != 0:
        raise DcclError(code, what)


def _torch():
    import torch
    return torch


def dtype_of(x):
    """ncclDataType_t value of a numpy array or torch tensor."""
    if isinstance(x, np.ndarray):
        return _NP_TO_DCCL[x.dtype]
    torch = _torch()
    table = {torch.int8: INT8, torch.uint8: UINT8, torch.int32: INT32, torch.int64: INT64, torch.float16: FLOAT16,
             torch.float32: FLOAT32, torch.float64: FLOAT64, torch.bfloat16: BFLOAT16}
    if hasattr(torch, "uint32"):
        table[torch.uint32] = UINT32
        table[torch.uint64] = UINT64
    return table[x.dtype]


def _addr(x):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("buffers must be contiguous")
        return x.ctypes.data
    if not x.is_contiguous():
        raise ValueError("buffers must be contiguous")
    return x.data_ptr()


def _numel(x):
    return x.size if isinstance(x, np.ndarray) else x.numel()


def _stream_of(x, stream):
    if stream is not None:
        return stream if isinstance(stream, int) else stream.cuda_stream
    if isinstance(x, np.ndarray):
        return None
    if x.is_cuda:
        return _torch().cuda.current_stream(x.device).cuda_stream
    return None


def get_unique_id():
    """128-byte rendezvous token; the calling process becomes the rendezvous server (rank 0)."""
    buf = ctypes.create_string_buffer(128)
    _check(lib().dccl_get_unique_id(buf), "dcclGetUniqueId")
    return buf.raw


class Communicator:
    """One rank's handle on a group of processes.

    ``Communicator()`` reads rank / world / rendezvous address from the
    environment or a configuration directory (see ``ncclCommInit``);
    ``Communicator(rank=, world=, unique_id=)`` takes them explicitly.
    ``device`` binds a CUDA device right away (a collective step: every rank
    passes its own device); without it the device side is set up by the first
    call that is given device memory.
    """

    def __init__(self, rank=None, world=None, unique_id=None, device=None):
        self._h = ctypes.c_void_p()
        if unique_id is not None:
            buf = ctypes.create_string_buffer(bytes(unique_id), 128)
            _check(lib().dccl_comm_init_rank(ctypes.byref(self._h), int(world), buf, int(rank)), "dcclCommInitRank")
        else:
            if rank is not None:
                os.environ["DCCL_RANK"] = str(rank)
                os.environ["DCCL_WORLD_SIZE"] = str(world)
            _check(lib().dccl_comm_init(ctypes.byref(self._h)), "ncclCommInit")
        self.rank = lib().dccl_rank(self._h)
        self.world = lib().dccl_world_size(self._h)
        if device is not None:
            _check(lib().dccl_comm_bind_device(self._h, int(device)), "device setup")

    @classmethod
    def from_handle(cls, handle):
        """Wrap a native communicator that something else owns (the PyTorch backend); finalize() is then a no-op."""
        self = cls.__new__(cls)
        self._h = ctypes.c_void_p(handle)
        self._borrowed = True
        self.rank = lib().dccl_rank(self._h)
        self.world = lib().dccl_world_size(self._h)
        return self

    def bind_device(self, device):
        """Set up the device side now (collective: every rank calls it with its own device)."""
        _check(lib().dccl_comm_bind_device(self._h, int(device)), "device setup")

    # -- life cycle ---------------------------------------------------
    def finalize(self):
        if getattr(self, "_borrowed", False):
            return
        if self._h:
            h, self._h = self._h, ctypes.c_void_p()
            _check(lib().dccl_comm_finalize(h), "ncclCommFinalize")

    def abort(self):
        _check(lib().dccl_comm_abort(self._h), "dcclCommAbort")

    def shrink(self, device=None):
        """After a failure: a new communicator over the ranks that are still there (every survivor calls it).
        This communicator stays usable for last_error() and should still be finalized."""
        new = Communicator.__new__(Communicator)
        new._h = ctypes.c_void_p()
        _check(lib().dccl_comm_shrink(self._h, ctypes.byref(new._h)), "dcclCommShrink")
        new.rank = lib().dccl_rank(new._h)
        new.world = lib().dccl_world_size(new._h)
        if device is not None:
            new.bind_device(device)
        return new

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finalize()

    def last_error(self):
        """(code, message) of the asynchronous state; code 0 means healthy."""
        code = ctypes.c_int(0)
        msg = ctypes.create_string_buffer(256)
        lib().dccl_last_error(self._h, ctypes.byref(code), msg, 256)
        return code.value, msg.value.decode()

    def check(self):
        code, msg = self.last_error()
        if code:
            raise DcclError(code, "communicator (" + msg + ")")

    @property
    def has_multicast(self):
        return bool(lib().dccl_has_multicast(self._h))

    @property
    def launches(self):
        return int(lib().dccl_launch_count(self._h))

    def topology(self):
        """The box as the communicator found it: {"nranks", "gpus": [...], "peer_access": [[...]], "peer_atomics": [[...]]}."""
        import json
        buf = ctypes.create_string_buffer(16384)
        _check(lib().dccl_topology_json(self._h, buf, len(buf)), "dcclGetTopology")
        return json.loads(buf.value.decode())

    def barrier(self):
        """Host-side barrier over the control plane (does not wait for CUDA streams)."""
        _check(lib().dccl_barrier(self._h), "dcclBarrier")

    def debug_check(self):
        """With DCCL_DEBUG_BOUNDS=1: raise when a kernel wrote into the unused parts of this rank's device pool
        (the message names the gap and the offset). No-op otherwise."""
        _check(lib().dccl_debug_check(self._h), "dcclDebugCheck")

    def stat(self, name):
        """A counter of the device side: "launches", "zero_copy_calls", "symmetric_calls" (calls that the peer kernels served straight out
        of / into user memory: symmetric, registered or lazily registered buffers)."""
        return int(lib().dccl_comm_stat(self._h, name.encode()))

    def set_param(self, name, value):
        """Tuning knob for sweeps: ctas (0 = table), threads, unroll, p2p_ctas, pipe_ctas, pipe_nv_ctas, pipe_chunk_kb,
        auto_register_min_kb (0: no lazy registration), direct_rs, direct_rooted, direct_rooted_ctas, direct_bcast_min_kb."""
        _check(lib().dccl_comm_set_param(self._h, name.encode(), int(value)), "set_param")

    def set_algorithm(self, collective, name):
        _check(lib().dccl_set_algorithm(self._h, collective.encode(), name.encode()), "dcclSetAlgorithm")

    def last_algorithm(self, collective):
        return lib().dccl_last_algorithm(self._h, collective.encode()).decode()

    # -- memory -------------------------------------------------------
    def register(self, x):
        nbytes = _numel(x) * DTYPE_SIZES[dtype_of(x)]
        _check(lib().dccl_register(self._h, _addr(x), nbytes), "dcclRegisterCacheMemory")

    def deregister(self, x):
        _check(lib().dccl_deregister(self._h, _addr(x)), "dcclDeregisterCacheMemory")

    def mem_alloc(self, nbytes):
        p = ctypes.c_void_p()
        _check(lib().dccl_mem_alloc(self._h, ctypes.byref(p), int(nbytes)), "dcclMemAlloc")
        return p.value

    def mem_free(self, ptr):
        _check(lib().dccl_mem_free(self._h, ctypes.c_void_p(ptr)), "dcclMemFree")

    def symmetric_empty(self, numel, dtype, device=None):
        """A torch tensor in symmetric (peer-mapped, multicast-bound) device memory. Collective.
        Free it with ``free_symmetric`` before the communicator is finalized."""
        from .utils.memory import tensor_from_pointer
        torch = _torch()
        itemsize = torch.empty((), dtype=dtype).element_size()
        ptr = self.mem_alloc(numel * itemsize)
        t = tensor_from_pointer(ptr, numel, dtype, device if device is not None else torch.cuda.current_device())
        t._dccl_ptr = ptr
        return t

    def free_symmetric(self, t):
        self.mem_free(t._dccl_ptr)

    def is_symmetric(self, t):
        """True when the tensor lies in symmetric memory of this communicator (``symmetric_empty`` or a pool from
        ``symmetric_mem_pool``): collectives on it need no staging copy and no registration."""
        return bool(lib().dccl_is_symmetric(self._h, _addr(t), _numel(t) * t.element_size()))

    def symmetric_mem_pool(self):
        """A ``torch.cuda.MemPool`` whose memory is symmetric (``dcclMemAlloc``): tensors created inside
        ``with torch.cuda.use_mem_pool(pool):`` (DDP's gradient buckets, activations that are reduced every step) are
        mapped by every rank and bound to the switch, so collectives on them run zero-copy without the code that
        allocates them knowing. Every rank must make the same allocations in the same order inside the pool. The memory
        is returned when the communicator is finalized. One communicator per process can serve pools at a time."""
        from . import _lib
        torch = _torch()
        lib().dccl_pool_bind(self._h)
        path = os.environ.get("DCCL_LIBRARY") or _lib.LIB_PATH
        self._pool_allocator = torch.cuda.memory.CUDAPluggableAllocator(path, "dccl_pool_alloc", "dccl_pool_free")
        return torch.cuda.MemPool(self._pool_allocator.allocator())

    # -- collectives --------------------------------------------------
    def all_reduce(self, send, recv=None, op="sum", stream=None):
        recv = send if recv is None else recv
        _check(lib().dccl_all_reduce(_addr(send), _addr(recv), _numel(send), dtype_of(send), OPS[op], self._h,
                                     _stream_of(send, stream)), "ncclAllReduce")
        return recv

    def reduce_scatter(self, send, recv, op="sum", stream=None):
        _check(lib().dccl_reduce_scatter(_addr(send), _addr(recv), _numel(recv), dtype_of(send), OPS[op], self._h,
                                         _stream_of(send, stream)), "ncclReduceScatter")
        return recv

    def all_gather(self, send, recv, stream=None):
        _check(lib().dccl_all_gather(_addr(send), _addr(recv), _numel(send), dtype_of(send), self._h,
                                     _stream_of(send, stream)), "ncclAllGather")
        return recv

    def broadcast(self, send, recv=None, root=0, stream=None):
        recv = send if recv is None else recv
        _check(lib().dccl_broadcast(_addr(send), _addr(recv), _numel(recv), dtype_of(recv), root, self._h,
                                    _stream_of(recv, stream)), "ncclBroadcast")
        return recv

    def reduce(self, send, recv=None, op="sum", root=0, stream=None):
        if recv is None and self.rank == root:
            recv = send
        _check(lib().dccl_reduce(_addr(send), _addr(recv), _numel(send), dtype_of(send), OPS[op], root, self._h,
                                 _stream_of(send, stream)), "ncclReduce")
        return recv

    def all_to_all(self, send, recv, send_counts=None, recv_counts=None, stream=None):
        """Block p of `send` goes to rank p, block p of `recv` comes from rank p. Equal blocks unless
        per-peer element counts are given (blocks are then packed back to back)."""
        if send_counts is None and recv_counts is None:
            _check(lib().dccl_all_to_all(_addr(send), _addr(recv), _numel(send) // self.world, dtype_of(send), self._h,
                                         _stream_of(send, stream)), "dcclAllToAll")
            return recv
        arr = ctypes.c_size_t * self.world
        sc = list(send_counts if send_counts is not None else [_numel(send) // self.world] * self.world)
        rc = list(recv_counts if recv_counts is not None else [_numel(recv) // self.world] * self.world)
        sd = [sum(sc[:p]) for p in range(self.world)]
        rd = [sum(rc[:p]) for p in range(self.world)]
        _check(lib().dccl_all_to_allv(_addr(send), arr(*sc), arr(*sd), _addr(recv), arr(*rc), arr(*rd), dtype_of(send), self._h,
                                      _stream_of(send, stream)), "dcclAllToAllv")
        return recv

    def gather(self, send, recv=None, root=0, stream=None):
        """The root receives every rank's `send` into block <rank> of `recv`."""
        _check(lib().dccl_gather(_addr(send), _addr(recv) if recv is not None else None, _numel(send), dtype_of(send), root, self._h,
                                 _stream_of(send, stream)), "dcclGather")
        return recv

    def scatter(self, send, recv, root=0, stream=None):
        """Rank p receives block p of the root's `send` into `recv`."""
        _check(lib().dccl_scatter(_addr(send) if send is not None else None, _addr(recv), _numel(recv), dtype_of(recv), root, self._h,
                                  _stream_of(recv, stream)), "dcclScatter")
        return recv

    def group_start(self):
        """Same as the module-level group_start() (groups are per thread, not per communicator)."""
        group_start()

    def group_end(self):
        group_end()

    def send(self, x, peer, stream=None):
        _check(lib().dccl_send(_addr(x), _numel(x), dtype_of(x), peer, self._h, _stream_of(x, stream)), "ncclSend")

    def recv(self, x, peer, stream=None):
        _check(lib().dccl_recv(_addr(x), _numel(x), dtype_of(x), peer, self._h, _stream_of(x, stream)), "ncclRecv")
        return x


def group_start():
    _check(lib().dccl_group_start(), "dcclGroupStart")


def group_end():
    _check(lib().dccl_group_end(), "dcclGroupEnd")
