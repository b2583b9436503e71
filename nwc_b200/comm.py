"""Exchange buffers of the tensor-parallel decode loop: one per rank, visible to every rank of the node over NVLink.

Each rank allocates its buffer through the library (plain device memory), the 64-byte CUDA IPC handles travel through
`torch.distributed.all_gather_object`, and every rank opens the handles of the others.  The buffers carry the ranks'
partial o / down outputs, the flags of both reduction protocols and the words of the sharded argmax (layout:
nwc_b200/csrc/nwc_comm.h)."""
import ctypes

import torch

from . import _lib as L


class PeerBuffers:
    def __init__(self, group, hidden: int):
        import torch.distributed as dist
        self.group, self.hidden = group, hidden
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8: raise ValueError("at most 8 tensor-parallel ranks (one node)")
        own = ctypes.c_void_p()
        err = L.lib.nwc_comm_alloc(ctypes.byref(own), hidden)
        if err: raise RuntimeError(f"nwc_comm_alloc error {err}")
        self.own = own.value
        handle = (ctypes.c_uint8 * 64)()
        err = L.lib.nwc_comm_export(ctypes.c_void_p(self.own), handle)
        if err: raise RuntimeError(f"nwc_comm_export error {err}")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.opened = []
        pointers = []
        for r, h in enumerate(handles):
            if r == self.rank: pointers.append(self.own); continue
            peer = ctypes.c_void_p()
            err = L.lib.nwc_comm_import((ctypes.c_uint8 * 64).from_buffer_copy(h), ctypes.byref(peer))
            if err: raise RuntimeError(f"nwc_comm_import error {err} (rank {r}: no peer access between the two GPUs?)")
            self.opened.append(peer.value); pointers.append(peer.value)
        self.table = (ctypes.c_void_p * self.world)(*pointers)      # host array the launches read
        self._io = {}
        torch.cuda.synchronize()
        dist.barrier(group=group)                                   # every buffer is zeroed and open before the first kernel

    def io(self, in_slot: int = -1, out_slot: int = -1):
        """nwc_fused_options argument of nwc_linear_fused_opt (kept alive by this object: the library reads it at launch time)."""
        key = (in_slot, out_slot)
        if key not in self._io:
            self._io[key] = L.FusedOptions(ctypes.cast(self.table, ctypes.c_void_p), self.rank, self.world, in_slot, out_slot, self.hidden)
        return ctypes.byref(self._io[key])

    def slot(self, i: int) -> ctypes.c_void_p:
        """Where this rank's row-parallel matvec writes its partial output (slot 0: o, slot 1: down)."""
        return ctypes.c_void_p(L.lib.nwc_comm_slot(ctypes.c_void_p(self.own), self.hidden, i))

    def allreduce_add_rmsnorm(self, slot, h_in, h_out, norm_w, eps, xn):
        err = L.lib.nwc_allreduce_add_rmsnorm(L.stream(), self.table, self.rank, self.world, slot, L.ptr(h_in), L.ptr(h_out), L.ptr(norm_w), eps,
                                              self.hidden, L.ptr(xn))
        if err: raise RuntimeError(f"nwc_allreduce_add_rmsnorm error {err}")

    def close(self):
        """Every rank must have finished its kernels (synchronise and barrier first)."""
        for p in self.opened: L.lib.nwc_comm_release(ctypes.c_void_p(p))
        self.opened = []
        if self.own: L.lib.nwc_comm_free(ctypes.c_void_p(self.own)); self.own = None
