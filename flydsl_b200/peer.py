"""Device buffers that every rank of a process group can address directly.

The expert-parallel layer lets stage 2 store each expert output row straight into the buffer
of the rank that owns the token (``flymoe_moe_gemm2_scatter_rows``).  That needs, on every
rank, the address under which each peer's buffer is mapped into this process.  Two ways to
get it, tried in this order:

* ``torch.distributed._symmetric_memory`` (one allocation per rank, exchanged and mapped by
  torch).  Multicast binding is switched off first: only plain peer stores are used here.
* CUDA IPC through torch's own tensor sharing (``torch.multiprocessing.reductions``), the
  handles travelling through ``all_gather_object``; peer access is then enabled explicitly.

Nothing here runs on the data path: the mapping is set up once per layer.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist


class PeerBuffers:
    """``nbytes`` of device memory on every rank; ``ptrs[r]`` is rank r's buffer as seen from here."""

    def __init__(self, nbytes: int, device: torch.device, group=None, prefer: str | None = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self.kind = None
        self._keep = []                                  # handles / mapped tensors that must stay alive
        prefer = prefer or os.environ.get("FLYMOE_PEER_BUFFERS", "symmetric_memory")
        order = ["symmetric_memory", "cuda_ipc"] if prefer != "cuda_ipc" else ["cuda_ipc", "symmetric_memory"]
        errors = []
        for kind in order:
            ok_local = True
            try:
                getattr(self, "_setup_" + kind)(device)
            except Exception as exc:                     # noqa: BLE001 - reported below if every way fails
                ok_local = False
                errors.append(f"{kind}: {type(exc).__name__}: {exc}")
            # every rank must end up with the same mechanism
            flag = torch.tensor([1 if ok_local else 0], dtype=torch.int32, device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if int(flag.item()) == 1:
                self.kind = kind
                break
            self._keep.clear()
        if self.kind is None:
            raise RuntimeError("no way to map peer buffers on this system: " + "; ".join(errors))

    # ------------------------------------------------------------------ mechanisms
    def _setup_symmetric_memory(self, device) -> None:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
        grp = self.group if self.group is not None else dist.group.WORLD
        handle = symm.rendezvous(t, grp)
        self.local = t
        self.ptrs = [int(p) for p in handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != t.data_ptr():
            raise RuntimeError("symmetric memory returned an unexpected pointer table")
        self._keep += [t, handle]

    def _setup_cuda_ipc(self, device) -> None:
        from torch.multiprocessing.reductions import reduce_tensor

        from . import _lib
        t = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        rebuild, args = reduce_tensor(t)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (rebuild, args, torch.cuda.current_device()), group=self.group)
        self.local = t
        self.ptrs = []
        lib = _lib.load()
        for r, (fn, a, peer_dev) in enumerate(gathered):
            if r == self.rank:
                self.ptrs.append(t.data_ptr())
                continue
            mapped = fn(*a)                               # opens the peer's allocation in this process
            self._keep.append(mapped)
            if peer_dev != torch.cuda.current_device():
                _lib.check(lib.flymoe_enable_peer_access(int(peer_dev)), "enable_peer_access")
            self.ptrs.append(mapped.data_ptr())
        self._keep.append(t)

    # ------------------------------------------------------------------ helpers
    def barrier(self, scratch: torch.Tensor) -> None:
        """Stream-ordered rendezvous (no host wait): every rank's earlier kernels have completed,
        and with them their stores into peers' buffers, before any rank's later kernels start."""
        dist.all_reduce(scratch, group=self.group)
