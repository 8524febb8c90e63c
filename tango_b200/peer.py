"""Exchange between the GPUs of one node over peer memory instead of NCCL (no counterpart in the reference).

Every rank allocates its shared buffers through the library (plain cudaMalloc), publishes their CUDA IPC handles
through the process group (host side, once), and maps the buffers of the other ranks with its own device current.
After that the data path uses no library call:

  * `max_scalar`    -- barrier + all-reduce(max) of one float in one tiny kernel (`tango_peer_sync`),
  * `quantize_push` -- the quantizer stores its int8 rows straight into the gathered table of every GPU
                       (`tango_quantize_push`, `tango_quantize_relu_grad_push`), followed by one `barrier`.

All kernels take addresses that never change, so a training step that uses them can be captured in a CUDA graph.
Waits on other GPUs are bounded on the device; `status()` reports an expired wait.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import config
from ._lib import TangoError, check, lib


class _RawCuda:
    """Exposes a raw device allocation through __cuda_array_interface__ so that torch can view it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|i1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SharedBuffer:
    """`nbytes` zero-filled bytes on this rank's GPU that every rank of the group maps (a collective, host side):
    `local` is a torch int8 view of this rank's buffer, `ptrs[r]` the address of rank r's buffer in THIS process."""

    def __init__(self, nbytes: int, rank: int, world: int, device: torch.device, group=None):
        self.rank, self.device = rank, device
        self.ptrs, self._own, self.local = [None] * world, 0, None
        ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        err = None
        with torch.cuda.device(device):
            try:
                check(lib.tango_peer_alloc(nbytes, ctypes.byref(ptr), handle), "peer_alloc")
                self._own = ptr.value
                self.ptrs[rank] = ptr.value
                torch.cuda.synchronize(device)
            except Exception as exc:                              # reported below, on every rank alike
                err = exc
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle) if err is None else None, group=group)
            if err is None and all(h is not None for h in handles):
                try:
                    for r in range(world):
                        if r == rank:
                            continue
                        remote = ctypes.c_void_p()
                        buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                        check(lib.tango_peer_open(buf, ctypes.byref(remote)), "peer_open")   # maps it for THIS device
                        self.ptrs[r] = remote.value
                except Exception as exc:
                    err = exc
            # every rank learns whether every rank succeeded, so that all of them raise (or none does)
            oks = [None] * world
            dist.all_gather_object(oks, err is None and all(p is not None for p in self.ptrs), group=group)
        if not all(oks):
            self.release()
            raise RuntimeError(f"peer-memory set-up failed on rank(s) {[r for r, ok in enumerate(oks) if not ok]}"
                               + (f": {err}" if err is not None else ""))
        self.local = torch.as_tensor(_RawCuda(ptr.value, nbytes), device=device)
        self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64, device=device)

    def unmap_peers(self):
        """First half of a release: closes this process's mappings of the other ranks' buffers."""
        with torch.cuda.device(self.device):
            for r, p in enumerate(self.ptrs):
                if r != self.rank and p:
                    lib.tango_peer_close(p)
        self.ptrs = [p if r == self.rank else None for r, p in enumerate(self.ptrs)]

    def free_own(self):
        """Second half: frees this rank's buffer.  CUDA IPC requires that every importer has closed its mapping
        first, so all ranks must have finished unmap_peers() (a barrier) before any of them calls this."""
        with torch.cuda.device(self.device):
            self.local = None
            if self._own:
                lib.tango_peer_free(self._own)
        self.ptrs, self._own = [], 0

    def release(self):
        """Unmap + free in one go: only for the error path of the constructor, where no peer holds a mapping of a
        buffer whose set-up failed half-way, or for single-process use."""
        self.unmap_peers()
        self.free_own()


class PeerTransport:
    """limit_ns bounds every wait for another GPU (default 2 s).  It is also the largest skew the ranks may have at a
    rendezvous: a rank that arrives later than this (first-step lazy loading on a busy host, a rank-0-only evaluation
    between two steps) makes the others give up, record TANGO_ETIMEOUT and carry on with what they have, which is then
    wrong.  `allreduce_grads(..., peer=...)` spreads the status word to all ranks once per step and
    `raise_if_expired()` turns it into an exception on every rank alike."""

    def __init__(self, rank: int, world: int, device: torch.device, group=None, limit_ns: int = 0):
        assert 1 <= world <= 64
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self.limit_ns = int(limit_ns)
        self.group_status = torch.zeros(1, dtype=torch.float32, device=device)   # sum over ranks of expired waits
        self._stream = lambda: torch.cuda.current_stream(device).cuda_stream
        # rendezvous words: 2 banks of `world` 64-bit words on every rank, written by everybody
        self._slots = SharedBuffer(2 * world * 8, rank, world, device, group)
        self._slot_ptrs = self._slots.ptrs_dev
        self._round = torch.zeros(1, dtype=torch.int64, device=device)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self._tables: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor, SharedBuffer]] = {}
        torch.cuda.synchronize(device)

    # ------------------------------------------------------------------------------------------------ rendezvous
    def max_scalar(self, value: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """All ranks' maximum of a non-negative 1-element fp32 tensor (None: barrier only)."""
        out = torch.empty(1, dtype=torch.float32, device=self.device) if value is not None else None
        with torch.cuda.device(self.device):
            check(lib.tango_peer_sync(self._slot_ptrs.data_ptr(), self.rank, self.world, self._round.data_ptr(),
                                      value.data_ptr() if value is not None else None,
                                      out.data_ptr() if out is not None else None, self._status.data_ptr(),
                                      self.limit_ns, self._stream()), "peer_sync")
        from . import kernels
        kernels.launch_counter[0] += 1
        return out

    def barrier(self) -> None:
        self.max_scalar(None)

    def status(self) -> int:
        """0, or TANGO_ETIMEOUT if a wait of THIS rank for another GPU expired since the last reset.  Synchronises."""
        return int(self._status.item())

    def status_word(self) -> torch.Tensor:
        """The sticky per-rank status word on the device (int32, 0 or TANGO_ETIMEOUT)."""
        return self._status

    def reset_status(self) -> None:
        self._status.zero_()
        self.group_status.zero_()

    def raise_if_expired(self) -> None:
        """Raises on every rank if any rank's rendezvous expired in a step whose gradients went through
        `allreduce_grads(..., peer=self)` (which spreads the status), or if this rank's own did.  Synchronises: call it
        where the loop reads the loss anyway."""
        if float(self.group_status.item()) != 0.0 or int(self._status.item()) != 0:
            raise TangoError("a bounded wait for another GPU expired: the gathered int8 tables or the agreed scales of "
                             "that step may be incomplete (raise PeerTransport.limit_ns if ranks legitimately skew)")

    def close(self) -> None:
        """Unmaps and frees every shared buffer (a collective: all ranks call it, with no kernel of theirs in flight).
        Tensors returned by `table()` must not be used afterwards."""
        torch.cuda.synchronize(self.device)
        bufs = [buf for _tab, _ptrs, buf in self._tables.values()] + ([self._slots] if self._slots is not None else [])
        if dist.is_initialized():
            dist.barrier(group=self.group)           # nobody launches anything that touches the buffers any more
        for buf in bufs:
            buf.unmap_peers()
        if dist.is_initialized():
            dist.barrier(group=self.group)           # every importer has closed its mappings: exporters may free
        for buf in bufs:
            buf.free_own()
        self._tables.clear()
        self._slots = None

    # ------------------------------------------------------------------------------------------------ gathered tables
    def table(self, key, rows: int, ld: int):
        """The gathered int8 table [rows, ld] registered under `key` (created and mapped on every rank at first use,
        a collective: all ranks must ask for the same keys in the same order, outside CUDA-graph capture).
        Returns (local table, device array of every rank's table address)."""
        ent = self._tables.get(key)
        if ent is None:
            buf = SharedBuffer(rows * ld, self.rank, self.world, self.device, self.group)
            ent = (buf.local.view(rows, ld), buf.ptrs_dev, buf)
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
