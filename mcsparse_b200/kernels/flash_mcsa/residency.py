"""Where the per-layer metadata of token-sparse attention lives between its uses.

Indices (up to 503 MB per layer at 40 heads x 768 groups x 4096 tokens) and the bias-correction residual (1 GB
per layer at that shape) are written on an anchor step and read once per later step.  On a 180 GB part a whole
model's worth usually stays in HBM, which is the default; next to a large checkpoint it may not, so either can be
kept in pinned host memory instead and brought back one layer ahead of its use, as the reference does
(mcsparse/kernels/flash_mcsa/token_sparse.py:313-487: ``offload_to_cpu`` / ``prefetch`` /
``_get_prefetched_indices`` for the indices, ``offload_residual_to_cpu`` / ``prefetch_residual`` /
``_get_residual_raw`` for the residual).  One class serves both here.
"""

from __future__ import annotations

from typing import Optional

import torch


class OffloadSlot:
    """One cached tensor that is either resident in HBM or parked in pinned host memory.

    ``store(t, offload=True)`` copies ``t`` to the host on a side stream and drops the device reference (the
    allocator gets the block back once the copy has run); ``prefetch()`` starts the copy back on another side
    stream; ``get()`` hands out a device tensor that is ready on the CURRENT stream: the resident one, the prefetched
    one (a hit: the stream waits for the copy's event, the host does not), or - nothing prefetched - a copy issued
    on the current stream itself (a miss: correct, but the consumer waits for PCIe).  The host copy stays
    authoritative; a prefetched device copy is handed out once and then forgotten.
    """

    def __init__(self):
        self.gpu: Optional[torch.Tensor] = None
        self.cpu: Optional[torch.Tensor] = None
        self.pref: Optional[torch.Tensor] = None
        self._ev_off = self._ev_pref = None
        self._s_off = self._s_pref = None
        self._device = None
        self.hits = self.misses = 0

    @property
    def present(self) -> bool:
        return self.gpu is not None or self.cpu is not None or self.pref is not None

    @property
    def offloaded(self) -> bool:
        return self.gpu is None and self.cpu is not None

    def clear(self) -> None:
        if self._ev_off is not None:
            self._ev_off.synchronize()          # the source of a pending device-to-host copy must outlive it
        self.gpu = self.cpu = self.pref = None
        self._ev_off = self._ev_pref = None

    def store(self, t: Optional[torch.Tensor], offload: bool = False) -> None:
        keep_cpu = self.cpu if (offload and t is not None and self.cpu is not None and self.cpu.shape == t.shape
                                and self.cpu.dtype == t.dtype) else None
        prev_pref_ev = self._ev_pref
        self.clear()
        if t is None:
            return
        if not isinstance(t, torch.Tensor) or not offload or not t.is_cuda:
            self.gpu = t.detach() if isinstance(t, torch.Tensor) else t
            return
        t = t.detach()
        dev = t.device
        self._device = dev
        if self._s_off is None:
            self._s_off = torch.cuda.Stream(device=dev)
        self.cpu = keep_cpu if keep_cpu is not None else torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        self._s_off.wait_stream(torch.cuda.current_stream(dev))
        if prev_pref_ev is not None:
            self._s_off.wait_event(prev_pref_ev)          # an earlier copy back may still be reading the pinned buffer
        with torch.cuda.stream(self._s_off):
            self.cpu.copy_(t, non_blocking=True)
            t.record_stream(self._s_off)
        self._ev_off = self._s_off.record_event()

    def prefetch(self) -> bool:
        """Start the copy back to the device.  True if a transfer was started."""
        if self.gpu is not None or self.pref is not None or self.cpu is None:
            return False
        dev = self._device
        if self._s_pref is None:
            self._s_pref = torch.cuda.Stream(device=dev)
        if self._ev_off is not None:
            self._s_pref.wait_event(self._ev_off)
        with torch.cuda.stream(self._s_pref):
            self.pref = self.cpu.to(dev, non_blocking=True)
        self._ev_pref = self._s_pref.record_event()
        return True

    def get(self) -> Optional[torch.Tensor]:
        if self.gpu is not None:
            return self.gpu
        if self.pref is not None:
            cur = torch.cuda.current_stream(self._device)
            if self._ev_pref is not None:
                cur.wait_event(self._ev_pref)
            t, self.pref = self.pref, None
            t.record_stream(cur)                          # allocated on the prefetch stream, consumed here
            self.hits += 1
            return t
        if self.cpu is None:
            return None
        cur = torch.cuda.current_stream(self._device)
        if self._ev_off is not None:
            cur.wait_event(self._ev_off)
        self.misses += 1
        return self.cpu.to(self._device, non_blocking=True)
