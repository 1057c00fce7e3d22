"""Wrapping raw device pointers (symmetric allocations) as torch tensors without a copy."""
import torch


class _RawCudaBuffer:
    """Object exposing ``__cuda_array_interface__`` for ``nbytes`` bytes at ``ptr``."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}


def tensor_from_pointer(ptr, numel, dtype, device):
    """A 1-D tensor of ``numel`` elements of ``dtype`` aliasing device memory at ``ptr``.
    The memory is owned by the caller (it must outlive the tensor)."""
    itemsize = torch.empty((), dtype=dtype).element_size()
    dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    raw = torch.as_tensor(_RawCudaBuffer(ptr, numel * itemsize), device=dev)
    return raw.view(dtype)
