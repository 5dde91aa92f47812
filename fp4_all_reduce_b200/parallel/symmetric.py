"""Peer-mapped window allocation for one-process-per-GPU groups.

`allocate_symmetric(nbytes, device, group)` returns `(local tensor, [device pointer to rank r's buffer
for every r], handle)`.  The memory is CUDA virtual-memory-management memory exported between the
processes of the group (PyTorch's symmetric-memory allocator with the "CUDA" backend: cuMemCreate +
handle exchange + cuMemMap of every peer's allocation); stores through a peer pointer travel over
NVLink / NVSwitch.  The handle must stay alive as long as the pointers are used.

The reference project obtains the same kind of pointers from NCCL 2.31's symmetric windows
(harness/fp4ar_bench.cu:387-392: ncclMemAlloc, ncclCommWindowRegister, ncclGetLsaDevicePointer); the NCCL
in this stack has no host-side peer-pointer query, hence the direct VMM route.
"""
from __future__ import annotations

import torch


def allocate_symmetric(nbytes: int, device: torch.device, group):
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    try:
        if symm.get_backend(device) != "CUDA":
            symm.set_backend("CUDA")
    except Exception:
        pass
    with torch.cuda.device(device):
        t = symm.empty(nbytes, dtype=torch.uint8, device=device)
        handle = symm.rendezvous(t, group=group)
    world = dist.get_world_size(group)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    if len(ptrs) != world:
        raise RuntimeError(f"symmetric rendezvous returned {len(ptrs)} pointers for {world} ranks")
    rank = dist.get_rank(group)
    if ptrs[rank] != t.data_ptr():
        raise RuntimeError("local symmetric pointer does not match the local tensor")
    return t, ptrs, handle


def multicast_pointer(handle) -> int:
    """Device pointer of the NVLS multicast mapping of the window, or 0 when the fabric offers none."""
    try:
        if not handle.has_multicast_support:
            return 0
    except Exception:
        pass
    try:
        return int(handle.multicast_ptr or 0)
    except Exception:
        return 0
