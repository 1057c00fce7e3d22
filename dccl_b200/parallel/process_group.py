"""``torch.distributed`` backend ``"dccl"``.

    import dccl_b200.parallel.process_group      # registers the backend
    torch.distributed.init_process_group("dccl", ...)

CPU tensors use the shared-memory host collectives, CUDA tensors the device
kernels (see csrc/torch/pg_dccl.cpp). ``communicator(pg)`` returns a
``dccl_b200.Communicator`` that shares the process group's native
communicator, e.g. for symmetric allocations or for choosing a variant.
"""
import importlib.util

import torch
import torch.distributed as dist

from . import backend_build

_ext = None


def extension():
    """The compiled backend module (built in-tree on first use)."""
    global _ext
    if _ext is None:
        path = backend_build.build()
        spec = importlib.util.spec_from_file_location("_dccl_torch", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ext = mod
    return _ext


def _create(store, rank, size, timeout):
    return extension().create_backend(store, rank, size, float(timeout.total_seconds()))


def register():
    if "dccl" not in getattr(dist.Backend, "backend_list", []):
        dist.Backend.register_backend("dccl", _create, devices=["cpu", "cuda"])


def communicator(group=None):
    """A Communicator object over the native communicator of a "dccl" process group (not owned: do not finalize it)."""
    from ..comm import Communicator
    group = group if group is not None else dist.group.WORLD
    backend = None
    for dev in ("cuda", "cpu"):
        try:
            backend = group._get_backend(torch.device(dev))
            break
        except Exception:
            continue
    if backend is None:
        raise RuntimeError("the group has no dccl backend")
    handle = extension().comm_handle(backend)
    return Communicator.from_handle(handle)


register()
