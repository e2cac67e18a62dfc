"""A device buffer that every rank of a single-node job can address: one cudaMalloc per rank, opened in every
other rank through CUDA IPC (the driver's peer mapping over NVLink; no collective library involved).

Used by the several-GPU form of the list launch (bonsai_b200_chain_create_tp): every rank allocates the same
layout -- the gathered outputs plus a 64-byte counter block -- and hands the kernel the base address of every
rank's copy.  No reference counterpart (the reference is single-GPU).
"""
import torch

COUNTER_BYTES = 64


def _rt():
    from cuda.bindings import runtime as rt
    return rt


def _check(res, what):
    err = res[0] if isinstance(res, tuple) else res
    if int(err) != 0:
        raise RuntimeError(f"{what} failed with CUDA error {int(err)}")
    return res[1] if isinstance(res, tuple) and len(res) > 1 else None


class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}


class PeerBuffer:
    """`nbytes` of zeroed device memory (plus the counter block behind it) on the current device, mapped into
    every rank of `dist`'s default group.  `tensor` is the local copy as a uint8 torch tensor; `ptrs[q]` is rank
    q's copy as addressed from this process; `counter_offset` is where the kernel's counters live."""

    def __init__(self, nbytes, dist, rank, world):
        rt = _rt()
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.counter_offset = self.nbytes
        total = self.nbytes + COUNTER_BYTES
        self.total_bytes = total
        self._rt, self.rank, self.world = rt, rank, world
        self._ptr = int(_check(rt.cudaMalloc(total), "cudaMalloc"))
        _check(rt.cudaMemset(self._ptr, 0, total), "cudaMemset")
        _check(rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
        handle = _check(rt.cudaIpcGetMemHandle(self._ptr), "cudaIpcGetMemHandle")
        mine = bytes(bytearray(handle.reserved))
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        self.ptrs, self._opened = [], []
        for q in range(world):
            if q == rank:
                self.ptrs.append(self._ptr)
                continue
            h = rt.cudaIpcMemHandle_t()
            h.reserved = list(everyone[q])
            p = int(_check(rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle"))
            self.ptrs.append(p)
            self._opened.append(p)
        self.tensor = torch.as_tensor(_Raw(self._ptr, self.nbytes), device="cuda")
        dist.barrier()          # nobody launches before every rank has zeroed and mapped

    def close(self, dist=None):
        if self._ptr is None:
            return
        if dist is not None:
            dist.barrier()      # nobody unmaps while a peer may still write
        for p in self._opened:
            self._rt.cudaIpcCloseMemHandle(p)
        self.tensor = None
        self._rt.cudaFree(self._ptr)
        self._ptr = None
