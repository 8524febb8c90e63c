"""Exchange between the GPUs of one node over peer memory instead of NCCL (no counterpart in the reference).

Every rank allocates its buffers with the PyTorch allocator, publishes CUDA IPC handles through the process group
(host side, once), and maps the buffers of the other ranks.  After that the data path uses no library call:

  * `max_scalar`    -- barrier + all-reduce(max) of one float in one tiny kernel (`tango_peer_sync`),
  * `quantize_push` -- the quantizer stores its int8 rows straight into the gathered table of every GPU
                       (`tango_quantize_push`, `tango_quantize_relu_grad_push`), followed by one `barrier`.

All kernels take addresses that never change, so a training step that uses them can be captured in a CUDA graph.
Waits on other GPUs are bounded on the device; `status()` reports an expired wait.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import config
from ._lib import check, lib


def _share(t: torch.Tensor):
    """Picklable CUDA IPC description of the storage behind `t`."""
    return t.untyped_storage()._share_cuda_()


def _open(handle, dtype: torch.dtype) -> torch.Tensor:
    """Flat tensor over a peer's storage, mapped into this process."""
    storage = torch.UntypedStorage._new_shared_cuda(*handle)
    return torch.empty(0, dtype=dtype, device=storage.device).set_(storage)


class PeerTransport:
    def __init__(self, rank: int, world: int, device: torch.device, group=None):
        assert 1 <= world <= 64
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self._stream = lambda: torch.cuda.current_stream(device).cuda_stream
        # rendezvous words: 2 banks of `world` 64-bit words on every rank, written by everybody
        self._slots = torch.zeros(2 * world, dtype=torch.int64, device=device)
        self._round = torch.zeros(1, dtype=torch.int64, device=device)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self._peer_slots = self._exchange(self._slots, torch.int64)
        self._slot_ptrs = torch.tensor([t.data_ptr() for t in self._peer_slots], dtype=torch.int64, device=device)
        self._tables: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor, list]] = {}
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _exchange(self, local: torch.Tensor, dtype: torch.dtype):
        """Publishes `local` and returns the list of every rank's tensor (own entry = `local` itself)."""
        handles = [None] * self.world
        dist.all_gather_object(handles, _share(local), group=self.group)
        tensors = [local if r == self.rank else _open(handles[r], dtype) for r in range(self.world)]
        with torch.cuda.device(self.device):
            for t in tensors:                      # kernels of this device will address the peers' memory directly
                if t.device != self.device:
                    check(lib.tango_enable_peer_access(t.device.index), "enable_peer_access")
        return tensors

    # ------------------------------------------------------------------------------------------------ rendezvous
    def max_scalar(self, value: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """All ranks' maximum of a non-negative 1-element fp32 tensor (None: barrier only)."""
        out = torch.empty(1, dtype=torch.float32, device=self.device) if value is not None else None
        with torch.cuda.device(self.device):
            check(lib.tango_peer_sync(self._slot_ptrs.data_ptr(), self.rank, self.world, self._round.data_ptr(),
                                      value.data_ptr() if value is not None else None,
                                      out.data_ptr() if out is not None else None, self._status.data_ptr(),
                                      self._stream()), "peer_sync")
        from . import kernels
        kernels.launch_counter[0] += 1
        return out

    def barrier(self) -> None:
        self.max_scalar(None)

    def status(self) -> int:
        """0, or TANGO_ETIMEOUT if a wait for another GPU expired."""
        return int(self._status.item())

    # ------------------------------------------------------------------------------------------------ gathered tables
    def table(self, key, rows: int, ld: int):
        """The gathered int8 table [rows, ld] registered under `key` (created and mapped on every rank at first use,
        a collective: all ranks must ask for the same keys in the same order, outside CUDA-graph capture).
        Returns (local table, device array of every rank's table address)."""
        ent = self._tables.get(key)
        if ent is None:
            local = torch.zeros((rows, ld), dtype=torch.int8, device=self.device)
            peers = self._exchange(local, torch.int8)
            ptrs = torch.tensor([t.data_ptr() for t in peers], dtype=torch.int64, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            ent = (local, ptrs, peers)
            self._tables[key] = ent
        assert ent[0].shape == (rows, ld), "a gathered table keeps its shape"
        return ent[0], ent[1]

    def quantize_push(self, x: torch.Tensor, scale: torch.Tensor, table_ptrs: torch.Tensor, row0: int, ld: int,
                      mode: int, seed: int, call: int, row_scale: Optional[torch.Tensor] = None) -> None:
        """int8(x * row_scale / scale) stored at rows [row0, row0 + len(x)) of every rank's table."""
        from . import kernels
        x2, rows, cols, ldx = kernels._matrix(x)
        step = config.step_counter()
        with torch.cuda.device(self.device):
            check(lib.tango_quantize_push(x2.data_ptr(), rows, cols, ldx,
                                          row_scale.data_ptr() if row_scale is not None else None, scale.data_ptr(),
                                          table_ptrs.data_ptr(), self.world, row0, ld, mode, seed, call,
                                          step.data_ptr() if step is not None else None, self._stream()),
                  "quantize_push")
        kernels.launch_counter[0] += 1

    def relu_grad_quantize_push(self, g: torch.Tensor, y: torch.Tensor, scale: torch.Tensor, table_ptrs: torch.Tensor,
                                row0: int, ld: int, mode: int, seed: int, call: int,
                                row_scale: Optional[torch.Tensor] = None) -> None:
        """int8((y > 0 ? g : 0) * row_scale / scale) stored at rows [row0, ...) of every rank's table."""
        from . import kernels
        g2, rows, cols, ldg = kernels._matrix(g)
        y2, _, _, ldy = kernels._matrix(y)
        step = config.step_counter()
        with torch.cuda.device(self.device):
            check(lib.tango_quantize_relu_grad_push(g2.data_ptr(), ldg, y2.data_ptr(), ldy, rows, cols,
                                                    row_scale.data_ptr() if row_scale is not None else None,
                                                    scale.data_ptr(), table_ptrs.data_ptr(), self.world, row0, ld,
                                                    mode, seed, call,
                                                    step.data_ptr() if step is not None else None, self._stream()),
                  "quantize_relu_grad_push")
        kernels.launch_counter[0] += 1
