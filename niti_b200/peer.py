"""Device memory that every rank of one node can address (CUDA IPC), for the data-parallel update kernel.

Each rank has the library allocate one zeroed arena of the same size (niti_peer_arena_create), the IPC handles go
round the process group, and every rank maps the others' arenas for kernels of ITS device (niti_peer_arena_open):
``PeerArena.ptrs[r]`` is the address of rank r's arena in THIS process.  Plain peer mappings only: the memory is
not bound to an NVLink multicast object.
"""
import ctypes
import socket

import torch
import torch.distributed as dist

from ._lib import lib, check


def _gpu_id(device):
    props = torch.cuda.get_device_properties(device)
    return str(getattr(props, "uuid", "")) or f"index{torch.device(device).index}"


def peers_on_one_node(device, group=None):
    """True when the ranks of `group` sit on different GPUs of one host that can all address each other: the
    condition for kernels of different ranks to wait on one another (never two ranks on one GPU)."""
    world = dist.get_world_size(group)
    me = (socket.gethostname(), _gpu_id(device), torch.cuda.device_count())
    every = [None] * world
    dist.all_gather_object(every, me, group=group)
    if len({h for h, _, _ in every}) != 1 or len({g for _, g, _ in every}) != world:
        return False
    if any(n < world for _, _, n in every):
        return False
    idx = torch.device(device).index
    ok = all(torch.cuda.can_device_access_peer(idx, j) for j in range(torch.cuda.device_count()) if j != idx)
    oks = [None] * world
    dist.all_gather_object(oks, bool(ok), group=group)
    return all(oks)


class _RawBytes:
    """Lets torch.as_tensor adopt library-owned device memory without a copy."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    def __init__(self, nbytes, device, group=None):
        self.device, self.group = torch.device(device), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self._own, self._mapped, self.ptrs, self.local, self.error = None, [], [], None, None
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            own = ctypes.c_void_p()
            try:
                check(lib.niti_peer_arena_create(self.nbytes, ctypes.byref(own), handle), "niti_peer_arena_create")
                self._own = own.value
            except Exception as e:  # reported below, after every rank has learnt of it
                self.error = e
            every = [None] * self.world
            dist.all_gather_object(every, (self._own is not None, handle.raw), group=group)
            if all(ok for ok, _ in every):
                for r, (_, raw) in enumerate(every):
                    if r == self.rank:
                        self.ptrs.append(self._own)
                        continue
                    try:
                        p = ctypes.c_void_p()
                        check(lib.niti_peer_arena_open(ctypes.create_string_buffer(raw, 64), ctypes.byref(p)), "niti_peer_arena_open")
                        self._mapped.append(p.value)
                        self.ptrs.append(p.value)
                    except Exception as e:
                        self.error = e
                        break
            oks = [None] * self.world
            dist.all_gather_object(oks, self.error is None and len(self.ptrs) == self.world, group=group)
        self.ok = all(oks)
        if not self.ok:
            self.close()
            return
        self.local = torch.as_tensor(_RawBytes(self._own, self.nbytes), device=self.device)
        dist.barrier(group)  # every arena is zeroed and mapped everywhere before anybody's kernel writes to one

    def view(self, offset, nbytes, dtype, shape=None):
        """A tensor over bytes [offset, offset + nbytes) of the OWN arena."""
        t = self.local[offset:offset + nbytes].view(dtype)
        return t if shape is None else t.view(shape)

    def close(self):
        """Unmap the peers' arenas, then free the own one; collective (an owner must outlive the mappings of its
        arena).  Tensors made by ``view`` must not be used afterwards."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._mapped:
                lib.niti_peer_arena_close(p)
            self._mapped, self.ptrs = [], []
            if dist.is_initialized():
                dist.barrier(self.group)
                torch.cuda.synchronize(self.device)
            if self._own is not None:
                self.local = None
                lib.niti_peer_arena_destroy(self._own)
                self._own = None
