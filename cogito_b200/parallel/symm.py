"""Symmetric device memory: a buffer of the same size on every rank of a group,
mapped into every rank's address space so that kernels can load from and store to a
peer's copy directly over NVLink.

Two providers, tried in this order:
  1. ``torch.distributed._symmetric_memory`` (CUDA driver VMM handles exchanged by
     the process group);
  2. CUDA IPC handles of an ordinary allocation, exchanged with ``all_gather_object``
     (what ``torch.multiprocessing`` uses to share CUDA tensors).
With a single rank the buffer is a plain local tensor.  Only kernels of this library
ever receive the peer addresses; no library kernel is given one.
"""
from __future__ import annotations

import os
import weakref

import torch
import torch.distributed as dist


GUARD_BYTES = 256
GUARD_PATTERN = 0xA5
_LIVE = weakref.WeakSet()     # every buffer of this process (for check_all_canaries)


def check_all_canaries() -> bool:
    """True when no live symmetric buffer of this process has a damaged guard region."""
    return all(b.check_canaries() for b in list(_LIVE))


class SymmetricBuffer:
    """``canary=True`` (or ``COGITO_SYMM_CANARY=1``) brackets the buffer with two 256-byte guard
    regions holding a fixed pattern; :meth:`check_canaries` tells whether any rank's kernel stored
    outside the usable range (peers write into this memory by address, so nothing else would
    notice).  ``local`` / ``ptrs`` always describe the usable range."""

    def __init__(self, nbytes: int, device, group=None, canary: bool | None = None):
        self.device = torch.device(device)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.group = group
        self.world = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        self._keep = []          # objects that keep peer mappings alive
        self.provider = "local"
        self.multicast_ptr = 0   # NVSwitch multicast address of the buffer, when the provider bound one
        if canary is None:
            canary = os.environ.get("COGITO_SYMM_CANARY", "0") not in ("", "0")
        self.guard = GUARD_BYTES if canary else 0
        usable, self.nbytes = self.nbytes, self.nbytes + 2 * self.guard     # providers allocate guards too
        try:
            self._allocate()
        finally:
            self.nbytes = usable
        self._raw = self.local
        _LIVE.add(self)
        if self.guard:
            self._raw[:self.guard] = GUARD_PATTERN
            self._raw[self.guard + usable:] = GUARD_PATTERN
            self.local = self._raw[self.guard:self.guard + usable]
            self.ptrs = [p + self.guard for p in self.ptrs]
            if self.multicast_ptr:
                self.multicast_ptr += self.guard
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(self.group)

    def check_canaries(self) -> bool:
        """True when both guard regions of the LOCAL copy still hold the pattern (always True
        without guards).  Call it after the kernels that use the buffer have finished."""
        if not self.guard:
            return True
        lo, hi = self._raw[:self.guard], self._raw[self.guard + self.nbytes:]
        return bool((lo == GUARD_PATTERN).all()) and bool((hi == GUARD_PATTERN).all())

    def _allocate(self):
        if self.world == 1:
            self.local = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.local.data_ptr()]
            return
        err = None
        if os.environ.get("COGITO_SYMM_PROVIDER", "symm") == "symm":
            try:
                self._init_symm_mem()
                return
            except Exception as e:  # fall through to IPC
                err = e
        try:
            self._init_ipc()
        except Exception as e2:
            raise RuntimeError(f"no symmetric-memory provider works here: symm_mem: {err!r}; ipc: {e2!r}")

    # -- provider 1 -------------------------------------------------------------
    def _init_symm_mem(self):
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        hdl = symm_mem.rendezvous(t, group=self.group)
        t.zero_()
        self.local = t
        self.ptrs = [int(p) for p in hdl.buffer_ptrs]
        try:
            self.multicast_ptr = int(getattr(hdl, "multicast_ptr", 0) or 0)
        except Exception:
            self.multicast_ptr = 0
        self._keep.append(hdl)
        self.provider = "symm_mem"
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # -- provider 2 -------------------------------------------------------------
    def _init_ipc(self):
        t = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize(self.device)
        handle = t.untyped_storage()._share_cuda_()
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=self.group)
        self.local = t
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(t.data_ptr())
                continue
            h = list(h)
            h[0] = self.device.index if self.device.index is not None else torch.cuda.current_device()
            st = torch.UntypedStorage._new_shared_cuda(*h)
            peer = torch.empty(0, dtype=torch.uint8, device=self.device).set_(st)
            self._keep.append(peer)
            self.ptrs.append(peer.data_ptr())
        self.provider = "cuda_ipc"
        dist.barrier(self.group)

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        """A typed view of the LOCAL copy starting at byte `offset`."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        if offset % 16 or offset + nbytes > self.nbytes:
            raise ValueError("view outside the buffer or misaligned")
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def peer_ptrs(self, offset: int = 0) -> list[int]:
        return [p + offset for p in self.ptrs]
