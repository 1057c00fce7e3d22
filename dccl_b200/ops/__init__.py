"""Differentiable collectives (``dccl_b200.ops.functional``)."""
from .functional import (all_gather, all_reduce, all_to_all, broadcast, copy_to_region, get_default_communicator,  # noqa: F401
                         recv, reduce_from_region, reduce_scatter, ring_shift, send, set_default_communicator)
