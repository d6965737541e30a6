"""Forward + backward of the scan for callers whose tensors live in HOST memory.

``HostPipeline.run`` takes pinned host buffers for x, dt, B, C, dy (and the per-head A_head, D), and writes
y, dx, ddt, dB, dC (and dA_head, dD) into pinned host buffers.  The batch is cut into micro-batches and three
CUDA streams overlap the host->device copies of micro-batch i+1, the kernels of micro-batch i and the
device->host copies of micro-batch i-1, so that a step costs about max(copy-in, compute, copy-out) instead
of their sum.  Batch entries are independent scans, so slicing the batch changes no result; the per-head
gradients dA_head and dD are summed over the micro-batches on the device.

This is the end-to-end path ``bench.py`` times (``e2e``): it goes through the public operator
(``ssd_mamba2``), i.e. through the C ABI, for every micro-batch.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .ssd_scan import ssd_mamba2

_IN = ("x", "dt", "B", "C", "dy")
_OUT = ("y", "dx", "ddt", "dB", "dC")


class HostPipeline:
    def __init__(self, device: torch.device | str = "cuda", micro_batches: int = 8):
        self.dev = torch.device(device)
        self.nmb = int(micro_batches)
        self.s_in = torch.cuda.Stream(self.dev)
        self.s_cmp = torch.cuda.Stream(self.dev)
        self.s_out = torch.cuda.Stream(self.dev)
        self._slots = None

    def _ensure_slots(self, host_in: dict[str, Tensor], mb: int) -> None:
        key = tuple((k, tuple(host_in[k].shape[1:]), host_in[k].dtype) for k in _IN) + (mb,)
        if self._slots is not None and self._slots[0] == key:
            return
        slots = [{k: torch.empty((mb,) + tuple(host_in[k].shape[1:]), dtype=host_in[k].dtype, device=self.dev)
                  for k in _IN} for _ in range(2)]
        self._slots = (key, slots)

    @staticmethod
    def alloc_outputs(host_in: dict[str, Tensor]) -> dict[str, Tensor]:
        """Pinned host buffers of the right shapes for ``run``'s results."""
        x, dt, B = host_in["x"], host_in["dt"], host_in["B"]
        h = x.shape[2]
        out = {"y": torch.empty_like(x), "dx": torch.empty_like(x), "ddt": torch.empty(dt.shape, dtype=torch.float32),
               "dB": torch.empty_like(B), "dC": torch.empty_like(B), "dA_head": torch.empty(h, dtype=torch.float32),
               "dD": torch.empty(h, dtype=torch.float32)}
        return {k: v.pin_memory() for k, v in out.items()}

    def run(self, host_in: dict[str, Tensor], host_out: dict[str, Tensor], chunk_size: int) -> None:
        """host_in: pinned x (b,T,h,p), dt (b,T,h), B, C (b,T,g,n), dy (b,T,h,p), A_head (h), D (h).
        Returns when every result is in host_out (the calling thread is synchronised with the copy-out stream)."""
        b = host_in["x"].shape[0]
        nmb = min(self.nmb, b)
        while b % nmb:
            nmb -= 1
        mb = b // nmb
        self._ensure_slots(host_in, mb)
        slots = self._slots[1]
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_cmp):
            A_head = host_in["A_head"].to(self.dev, non_blocking=True).requires_grad_(True)
            D = host_in["D"].to(self.dev, non_blocking=True).requires_grad_(True)
            dAh = torch.zeros_like(A_head)
            dD = torch.zeros_like(D)
        ev_in = [torch.cuda.Event() for _ in range(nmb)]
        ev_cmp = [torch.cuda.Event() for _ in range(nmb)]
        for i in range(nmb):
            sl = slice(i * mb, (i + 1) * mb)
            slot = slots[i % 2]
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(ev_cmp[i - 2])  # the kernels of micro-batch i-2 are done with this slot
                for k in _IN:
                    slot[k].copy_(host_in[k][sl], non_blocking=True)
                ev_in[i].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ev_in[i])
                x = slot["x"].detach().requires_grad_(True)
                dt = slot["dt"].detach().requires_grad_(True)
                Bm = slot["B"].detach().requires_grad_(True)
                Cm = slot["C"].detach().requires_grad_(True)
                y, _ = ssd_mamba2(x, dt, A_head, Bm, Cm, D, chunk_size)
                gx, gdt, gA, gB, gC, gD = torch.autograd.grad([y], [x, dt, A_head, Bm, Cm, D], [slot["dy"]])
                dAh += gA
                dD += gD
                res = {"y": y.detach(), "dx": gx, "ddt": gdt, "dB": gB, "dC": gC}
                ev_cmp[i].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_cmp[i])
                for k in _OUT:
                    res[k].record_stream(self.s_out)
                    host_out[k][sl].copy_(res[k], non_blocking=True)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_stream(self.s_cmp)
            dAh.record_stream(self.s_out)
            dD.record_stream(self.s_out)
            host_out["dA_head"].copy_(dAh, non_blocking=True)
            host_out["dD"].copy_(dD, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_cmp)
        cur.wait_stream(self.s_in)
