"""dccl_b200: Blackwell-native collective communication with the DCCL / NCCL-style API.

    from dccl_b200 import Communicator
    comm = Communicator()                # rank / world from the environment
    comm.all_reduce(tensor, op="avg")    # torch CUDA tensor: one sm_100a kernel on the current stream
    comm.all_reduce(array)               # numpy array: shared-memory host path

The native library (``libdccl.so``) carries the whole implementation; this
package binds it, adds the PyTorch process group and DDP communication hook
(``dccl_b200.parallel``) and the model used by the training benchmark
(``dccl_b200.models``).
"""
from .comm import (AVG, BFLOAT16, FLOAT16, FLOAT32, FLOAT64, INT8, INT32, INT64, MAX, MIN, PROD, SUM, UINT8, UINT32,  # noqa: F401
                   UINT64, Communicator, DcclError, get_unique_id, group_end, group_start)
from ._lib import LIB_PATH, build, lib  # noqa: F401

__all__ = ["Communicator", "DcclError", "get_unique_id", "group_start", "group_end", "build", "lib", "LIB_PATH"]
