"""The activation all-reduce of the partitioned mode in one kernel over NVLink peer memory.

After every row-parallel layer the ranks' partial outputs are summed: a ``[batch, hidden]`` BF16
tensor, 32 KB at batch 1 for hidden 16384.  A library collective is pure latency at that size
(19-22 microseconds each through NCCL at two and four ranks when nothing runs between them, two
per transformer layer; this kernel: 4.3).
``df11_allreduce_bf16`` (``csrc/df11_allreduce.cu``) does it in one launch with plain peer loads
and stores on buffers that every rank can address (up to 64 KB: every rank pushes its slice to
all ranks as tagged 8-byte pairs, one NVLink crossing); this module sets those buffers up with
torch's symmetric memory and keeps one set per process group and device.  The reference has no
such mode at all (its only multi-GPU form places whole layers on different devices,
dfloat11/dfloat11.py:455-460).

Used by the partitioned mode unless ``DF11_PEER_ALLREDUCE=0`` (read when ``apply_tensor_parallel``
runs).  Whatever cannot go through the kernel -- another dtype, more than ``SLOT_BYTES``, a set-up
that failed on any rank -- goes through ``torch.distributed.all_reduce``; compare models only with
the same setting, the two ways of summing round differently.  A call that gives up waiting for a
peer (``DF11_ALLREDUCE_WAIT_MS``, 30 s) sets a status word, after which further calls return at
once; ``dfloat11_b200.check_status()`` raises on it.
"""
from __future__ import annotations

import ctypes
import logging
from typing import Dict, Optional

import torch

from . import _lib

log = logging.getLogger("dfloat11")

SLOT_BYTES = 1 << 20          # largest tensor the kernel takes (batch 32 at hidden 16384)


class PeerAllReduce:
    """Buffers, flags and the call counter of one process group on one device."""

    _instances: Dict[tuple, Optional["PeerAllReduce"]] = {}

    def __init__(self, group, device: torch.device, slot_bytes: int = SLOT_BYTES):
        import os
        import torch.distributed as dist
        # The kernel uses plain peer loads and stores only.  Binding the buffers to an NVLink
        # multicast object as well (what the symmetric-memory rendezvous does when the hardware
        # offers it) would buy nothing here and ties the ranks' memory together beyond the life
        # of a single rank, so it is switched off unless the caller has decided otherwise.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise RuntimeError("the peer all-reduce handles up to 8 ranks")
        self.device = device
        self.slot_bytes = int(slot_bytes)
        flag_bytes = int(_lib.lib.df11_allreduce_flag_bytes())
        self.buffer = symm_mem.empty(2 * self.slot_bytes + flag_bytes, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
        try:
            self.multicast_bound = bool(self.handle.multicast_ptr)      # 0 when no multicast object was made
        except Exception:  # noqa: BLE001 - informational only
            self.multicast_bound = None
        pointers = [int(p) for p in self.handle.buffer_ptrs]
        self._data = (ctypes.c_uint64 * 8)(*(pointers + [0] * (8 - len(pointers))))
        self._flags = (ctypes.c_uint64 * 8)(*([p + 2 * self.slot_bytes for p in pointers] + [0] * (8 - len(pointers))))
        self.counters = torch.zeros(int(_lib.lib.df11_allreduce_counter_bytes()) // 4, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        # How long a rank waits for the others inside one call.  Ranks of a serving job run in step,
        # but a host may stall one of them for seconds (a collection pause, a log write); a library
        # collective would simply wait.  After the first call that gave up the others return at once.
        self.wait_ms = int(os.environ.get("DF11_ALLREDUCE_WAIT_MS", "30000"))
        self.calls = 0
        # nobody writes a flag before every rank's flag area is zero
        dist.barrier(group=group, device_ids=[device.index])
        torch.cuda.synchronize(device)

    @classmethod
    def get(cls, group, device: torch.device) -> Optional["PeerAllReduce"]:
        """The instance for (group, device), made on first use by all ranks together; None when
        symmetric memory cannot be set up here (logged once; the caller uses the library collective)."""
        key = (id(group) if group is not None else None, device)
        if key not in cls._instances:
            import torch.distributed as dist
            try:
                instance = cls(group, device)
            except Exception as exc:  # noqa: BLE001 - optional acceleration
                log.warning("peer all-reduce unavailable (%s: %s); using torch.distributed.all_reduce",
                            type(exc).__name__, exc)
                instance = None
            # all ranks or none: a rank that summed through the library while its peers wait in the
            # kernel would leave them waiting
            agreed = torch.tensor([int(instance is not None)], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            cls._instances[key] = instance if int(agreed.item()) else None
        return cls._instances[key]

    def all_reduce_(self, tensor: torch.Tensor) -> bool:
        """Sums ``tensor`` over the ranks in place; False if this tensor is not one the kernel takes."""
        if (tensor.dtype != torch.bfloat16 or not tensor.is_cuda or tensor.device != self.device
                or not tensor.is_contiguous() or tensor.numel() % 8 or tensor.numel() * 2 > self.slot_bytes
                or tensor.data_ptr() % 16):
            return False
        _lib.check(_lib.lib.df11_allreduce_bf16(
            self._data, self._flags, self.counters.data_ptr(), self.rank, self.world, tensor.data_ptr(),
            tensor.data_ptr(), tensor.numel(), self.slot_bytes, self.wait_ms, self.status.data_ptr(), self.device.index,
            torch.cuda.current_stream(self.device).cuda_stream))
        self.calls += 1
        return True

    def check(self) -> None:
        """Raises if a call gave up waiting for a peer (synchronises)."""
        if int(self.status.item()):
            self.status.zero_()
            raise _lib.DF11Error(_lib.DF11_ERR_CUDA, "a peer all-reduce timed out waiting for another rank")
