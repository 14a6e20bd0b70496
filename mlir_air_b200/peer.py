"""Send buffers and flag words that every tensor-parallel rank can reach: the host side of the
peer-memory hand-over (awq_b200_gemv_f32_push / awq_b200_tp_reduce_add_rmsnorm_act).

The counterpart of the reference's symmetric heap (runtime_lib/airgpu/symmetric_heap.cpp:172-312:
every rank allocates the same buffer, exports it, and maps all peers' buffers into its own address
space).  Here the mapping comes from torch's symmetric memory, or, where that is unavailable, from
CUDA IPC handles exchanged over the process group.  One process per GPU, one node.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch
import torch.distributed as dist

FLAG_WORDS = 16          # uint32 per slot: [0, 8) arrivals per sender, [8] blocks done, rest unused
FLAG_BYTES = 256         # the flag block of a slot, padded


def _map_with_symmetric_memory(nbytes: int, device, group):
    import torch.distributed._symmetric_memory as symm
    name = group.group_name if hasattr(group, "group_name") else group
    try:
        symm.enable_symm_mem_for_group(name)
    except Exception:
        pass  # newer releases enable it on first use
    buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    torch.cuda.synchronize(device)
    hdl = symm.rendezvous(buf, name)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    return buf, ptrs, [hdl]


def _map_with_ipc(nbytes: int, device, group):
    from torch.multiprocessing.reductions import reduce_tensor
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    torch.cuda.synchronize(device)
    gathered = [None] * world
    dist.all_gather_object(gathered, reduce_tensor(buf), group=group)
    keep, ptrs = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(buf.data_ptr())
            continue
        fn, args = gathered[r]
        t = fn(*args)  # a tensor on the owner's device, mapped into this process
        # kernels on this GPU dereference the pointer: peer access must be on for the pair
        torch.empty(1, device=t.device).to(device)
        keep.append(t)
        ptrs.append(t.data_ptr())
    return buf, ptrs, keep


class PeerBuffers:
    """`n_slots` send slots of `recv_bytes` bytes (+ a flag block each) on every rank of `group`,
    all of them addressable from this GPU.  Slot s of rank r: partial at ptrs[r] + s * stride, flags
    behind it."""

    def __init__(self, group, n_slots: int, recv_bytes: int, device):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.n_slots = n_slots
        self.recv_bytes = (recv_bytes + 255) // 256 * 256
        self.stride = self.recv_bytes + FLAG_BYTES
        total = n_slots * self.stride
        device = torch.device(device)
        try:
            self.buf, self.ptrs, self._keep = _map_with_symmetric_memory(total, device, group)
            self.how = "symmetric_memory"
        except Exception as e:  # noqa: BLE001 -- any failure of the experimental API: fall back to IPC
            self._symm_error = repr(e)
            self.buf, self.ptrs, self._keep = _map_with_ipc(total, device, group)
            self.how = "cuda_ipc"
        dist.barrier(group=group)
        arr = ctypes.c_void_p * self.world
        self._recv_arrays = [arr(*[p + s * self.stride for p in self.ptrs]) for s in range(n_slots)]
        self._flag_arrays = [arr(*[p + s * self.stride + self.recv_bytes for p in self.ptrs]) for s in range(n_slots)]

    def reset(self):
        """Collective: zero this rank's slots, flags and launch count, on every rank, with nothing in flight.  To be
        called by all ranks after any of them saw a launch fail (a device-side wait that gave up, an argument error on
        one rank only): the in-kernel exchange numbers its messages by the launches that finished on a rank, and ranks
        that disagree about that number would wait for each other's messages in vain.  A peer buffer also belongs to
        one plan (one layer count): the message numbers of a launch are launches x layers + layer."""
        torch.cuda.synchronize(self.buf.device)
        dist.barrier(group=self.group)
        self.buf.zero_()
        torch.cuda.synchronize(self.buf.device)
        dist.barrier(group=self.group)

    def base_array(self):
        """ctypes array of every rank's buffer base (argument peer_base)."""
        return self._recv_arrays[0]

    def send_array(self, slot: int):
        """ctypes array of every rank's send-buffer pointer for `slot` (argument peer_partials)."""
        return self._recv_arrays[slot]

    def flag_array(self, slot: int):
        return self._flag_arrays[slot]

    def local_send(self, slot: int) -> int:
        return self.ptrs[self.rank] + slot * self.stride

    def local_flags(self, slot: int) -> int:
        return self.local_send(slot) + self.recv_bytes
