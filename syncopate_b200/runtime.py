"""Process-level runtime: one process per GPU, symmetric buffers over CUDA IPC.

Replaces what the reference gets from ``triton_dist`` + NVSHMEM (``initialize_distributed``,
``nvshmem_create_tensors``, ``nvshmem_barrier_all_on_stream``; e.g. tests/test_ag_gemm_gen.py:83,
communication_context.py:38-62).  ``torch.distributed`` is used for plumbing only (agreeing on a
rendezvous directory, test-time reductions); no collective library call sits on the fused path.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import tempfile
import uuid
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib as L


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 2,
        }


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A torch view (no ownership) of ``shape`` x ``dtype`` at device address ``ptr``."""
    n = 1
    for d in shape:
        n *= int(d)
    nbytes = max(n * dtype.itemsize, 1)
    flat = torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)
    return flat[: n * dtype.itemsize].view(dtype).view(*shape)


class SymmetricTensor:
    """One symmetric allocation: ``local`` tensor, ``peers[r]`` views, and the C table ``symm``."""

    def __init__(self, symm: L.Symm, shape, dtype, device):
        self.symm = symm
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype
        self.peers: List[torch.Tensor] = [
            tensor_from_ptr(symm.ptrs[r], self.shape, dtype, device) for r in range(symm.world)
        ]
        self.local = self.peers[symm.rank]


_CURRENT = None  # the context most recently opened in this process


def current_context():
    """The process's symmetric context: the one ``init_from_env`` (or the latest ``SymmetricContext``
    constructor) opened.  Plays the role of the reference's process-wide NVSHMEM heap, which its
    ``CommContext(rank, info)`` allocates from without being handed anything."""
    if _CURRENT is None:
        raise RuntimeError("no symmetric context is open in this process: call "
                           "syncopate_b200.runtime.init_from_env() (one process per GPU) first")
    return _CURRENT


class SymmetricContext:
    """Owner of this rank's ``syn_ctx``."""

    def __init__(self, rank: int, world: int, device: Optional[int] = None, rendezvous_dir: Optional[str] = None):
        global _CURRENT
        _CURRENT = self
        self.rank, self.world = rank, world
        self.device_index = torch.cuda.current_device() if device is None else device
        self.device = torch.device("cuda", self.device_index)
        self._handle = C.c_void_p()
        self._dir = rendezvous_dir
        rdv = rendezvous_dir.encode() if rendezvous_dir else None
        L.check(L.lib().syn_ctx_create(rank, world, self.device_index, rdv, C.byref(self._handle)), "syn_ctx_create")
        self._closed = False
        self._allocs: List[SymmetricTensor] = []
        self.status = tensor_from_ptr(L.lib().syn_ctx_status_ptr(self._handle), (4,), torch.int32, self.device)

    def alloc(self, shape, dtype: torch.dtype, timeout_s: int = 0) -> SymmetricTensor:
        n = 1
        for d in shape:
            n *= int(d)
        symm = L.Symm()
        L.check(
            L.lib().syn_symm_alloc(self._handle, max(n * dtype.itemsize, 16), timeout_s, C.byref(symm)),
            "syn_symm_alloc",
        )
        t = SymmetricTensor(symm, shape, dtype, self.device)
        self._allocs.append(t)
        return t

    def barrier(self, stream: Optional[torch.cuda.Stream] = None, timeout_ns: int = 0) -> None:
        s = (stream or torch.cuda.current_stream()).cuda_stream or None
        L.check(L.lib().syn_barrier(self._handle, s, timeout_ns), "syn_barrier")

    def check(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Synchronises ``stream`` and raises if any kernel given this context's status block
        recorded a timed-out wait."""
        s = (stream or torch.cuda.current_stream()).cuda_stream or None
        words = (C.c_int32 * 4)()
        rc = L.lib().syn_ctx_status(self._handle, s, words)
        if rc != 0:
            raise L.SynError(rc, "device status", f"wave={words[1]} flag={words[2]} block={words[3]}")

    def close(self) -> None:
        """Collective: every rank calls it, after its last kernel that touches a peer has been
        issued.  The ranks meet at a device barrier first, so that no rank unmaps or frees a buffer
        that a peer's kernel may still be using."""
        global _CURRENT
        if not self._closed:
            self._closed = True
            if _CURRENT is self:
                _CURRENT = None
            if self.world > 1:
                try:
                    self.barrier()
                    torch.cuda.synchronize(self.device)
                except Exception:
                    pass
            self._allocs.clear()
            L.lib().syn_ctx_destroy(self._handle)
            if self._dir and self.rank == 0:
                shutil.rmtree(self._dir, ignore_errors=True)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class EmulatedWorld:
    """All ranks of a plan inside one process on one GPU: every "symmetric" allocation is a set of
    ``world`` ordinary device tensors and each rank's table holds their addresses.  For one-GPU
    tests of the fused kernels (a rank's launch may only depend on data and flags that earlier
    launches left behind, never on a kernel that has not run yet)."""

    def __init__(self, world: int, device: Optional[int] = None):
        self.world = world
        self.device_index = torch.cuda.current_device() if device is None else device
        self.device = torch.device("cuda", self.device_index)
        self._allocs: List[List[torch.Tensor]] = []
        self.contexts = [EmulatedContext(self, r) for r in range(world)]

    def _get(self, index: int, shape, dtype) -> List[torch.Tensor]:
        if index == len(self._allocs):
            self._allocs.append([torch.zeros(*shape, dtype=dtype, device=self.device) for _ in range(self.world)])
        group = self._allocs[index]
        if tuple(group[0].shape) != tuple(shape) or group[0].dtype != dtype:
            raise RuntimeError("ranks of an emulated world must allocate the same sequence of buffers")
        return group


class EmulatedContext:
    """One rank of an :class:`EmulatedWorld`; same surface as :class:`SymmetricContext`."""

    def __init__(self, world: EmulatedWorld, rank: int):
        self._world = world
        self.rank, self.world = rank, world.world
        self.device_index, self.device = world.device_index, world.device
        self._next = 0
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)

    def alloc(self, shape, dtype: torch.dtype, timeout_s: int = 0) -> SymmetricTensor:
        group = self._world._get(self._next, tuple(int(s) for s in shape), dtype)
        self._next += 1
        return SymmetricTensor(L.Symm.of(self.rank, [t.data_ptr() for t in group]), shape, dtype, self.device)

    def barrier(self, stream=None, timeout_ns: int = 0) -> None:
        torch.cuda.synchronize()

    def check(self, stream=None) -> None:
        torch.cuda.synchronize()
        words = self.status.tolist()
        if words[0] != 0:
            self.status.zero_()
            code = {1: -4, 2: -5, 3: -6}.get(words[0], -1)
            raise L.SynError(code, "device status", f"wave={words[1]} flag={words[2]} block={words[3]}")

    def close(self) -> None:
        pass


def init_from_env(backend: Optional[str] = None) -> Tuple[int, int, SymmetricContext]:
    """Launcher glue for ``torchrun`` (replaces utils/launch.sh + ``initialize_distributed``): reads
    RANK / LOCAL_RANK / WORLD_SIZE, binds the GPU, initialises ``torch.distributed`` when more than
    one rank runs (for plumbing), agrees on a fresh rendezvous directory and opens the symmetric
    context.  Returns ``(rank, world, context)``."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local_rank)
    rdv = None
    if world > 1:
        import torch.distributed as dist

        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend=backend or "nccl", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", local_rank))
        box = [None]
        if rank == 0:
            base = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
            box[0] = os.path.join(base, f"syncopate_b200_{uuid.uuid4().hex}")
            os.makedirs(box[0], exist_ok=True)
        dist.broadcast_object_list(box, src=0)
        rdv = box[0]
    ctx = SymmetricContext(rank, world, local_rank, rdv)
    return rank, world, ctx
