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

    def run(self, host_in: dict[str, Tensor], host_out: dict[str, Tensor], chunk_size: int, wait: bool = True):
        """host_in: pinned x (b,T,h,p), dt (b,T,h), B, C (b,T,g,n), dy (b,T,h,p), A_head (h), D (h).
        With ``wait`` (default) the calling THREAD blocks until every result is in host_out, so the host may read
        the buffers right after the call.  With ``wait=False`` the call returns at once with a CUDA event that
        completes when the last copy has landed; host_out must not be read before ``event.synchronize()``."""
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
        done = torch.cuda.Event()
        done.record(self.s_out)  # s_out is ordered after the kernels, which are ordered after the copies in
        if wait:
            done.synchronize()
            return None
        return done


class SequenceStreamer:
    """Forward + backward of the scan over a LONG sequence held in pinned host memory, one slice of the sequence
    on the GPU at a time, exact across slices: the state leaving a slice enters the next one
    (``initial_states`` / ``final_state`` of the operator), and in the backward the gradient of a slice's initial
    state is the next-earlier slice's final-state gradient.  The reference's streaming runner cuts the sequence
    the same way but lets every slice start from a zero state (src/runtime/chunked_offload.py:117-150); carrying
    the state makes the sliced result equal to the one-call result.

    GPU memory is independent of the sequence length: two input slots, one slice of results, and the small
    boundary states ((b,h,p,n) fp32 per slice).  Copies of slice s+1 overlap the kernels of slice s on a second
    stream.  The backward recomputes each slice's forward from its stored entering state (input-only
    checkpointing at slice granularity), walking the slices in reverse.
    """

    def __init__(self, device: torch.device | str = "cuda", slice_len: int = 4096):
        self.dev = torch.device(device)
        self.slice_len = int(slice_len)
        self.s_copy = torch.cuda.Stream(self.dev)
        self.s_out = torch.cuda.Stream(self.dev)

    def _load(self, host_in, names, s, slots, ev_free):
        sl = slice(s * self.slice_len, (s + 1) * self.slice_len)
        slot = slots[s % 2]
        with torch.cuda.stream(self.s_copy):
            if ev_free[s % 2] is not None:
                self.s_copy.wait_event(ev_free[s % 2])
            for k in names:
                slot[k].copy_(host_in[k][:, sl], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.s_copy)
        return slot, ev

    def run(self, host_in: dict[str, Tensor], host_out: dict[str, Tensor], chunk_size: int) -> None:
        """host_in: pinned x (b,T,h,p), dt (b,T,h), B, C (b,T,g,n), dy (b,T,h,p), A_head (h), D (h).  host_out: pinned
        y, dx, ddt, dB, dC, dA_head, dD (``HostPipeline.alloc_outputs``).  The calling thread blocks until every
        result is in host_out."""
        T = host_in["x"].shape[1]
        L = self.slice_len
        assert T % L == 0 and L % chunk_size == 0, f"sequence {T} / slice {L} / chunk {chunk_size} do not divide"
        ns = T // L
        dev = self.dev
        cur = torch.cuda.current_stream(dev)
        self.s_copy.wait_stream(cur)
        self.s_out.wait_stream(cur)
        A_head = host_in["A_head"].to(dev, non_blocking=True)
        D = host_in["D"].to(dev, non_blocking=True)
        b = host_in["x"].shape[0]

        def new_slots(names):
            return [{k: torch.empty((b, L) + tuple(host_in[k].shape[2:]), dtype=host_in[k].dtype, device=dev)
                     for k in names} for _ in range(2)]

        # ---- forward over the slices: y out, the state entering every slice kept on the GPU
        fwd_names = ("x", "dt", "B", "C")
        slots = new_slots(fwd_names)
        ev_free = [None, None]
        states = [None] * (ns + 1)
        nxt = self._load(host_in, fwd_names, 0, slots, ev_free)
        for s in range(ns):
            slot, ev = nxt
            if s + 1 < ns:
                nxt = self._load(host_in, fwd_names, s + 1, slots, ev_free)
            cur.wait_event(ev)
            with torch.no_grad():
                y, final = ssd_mamba2(slot["x"], slot["dt"], A_head, slot["B"], slot["C"], D, chunk_size, states[s])
            states[s + 1] = final
            done = torch.cuda.Event()
            done.record(cur)
            ev_free[s % 2] = done
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                y.record_stream(self.s_out)
                host_out["y"][:, s * L:(s + 1) * L].copy_(y, non_blocking=True)
        # ---- backward over the slices in reverse: recompute the slice from its entering state, pass d(state) on
        bwd_names = ("x", "dt", "B", "C", "dy")
        slots = new_slots(bwd_names)
        ev_free = [None, None]
        order = list(range(ns - 1, -1, -1))
        dAh = torch.zeros_like(A_head, dtype=torch.float32)
        dD = torch.zeros_like(D, dtype=torch.float32)
        dstate = None
        # slot parity follows the position in the reverse order
        def load_rev(i):
            s = order[i]
            sl = slice(s * L, (s + 1) * L)
            slot = slots[i % 2]
            with torch.cuda.stream(self.s_copy):
                if ev_free[i % 2] is not None:
                    self.s_copy.wait_event(ev_free[i % 2])
                for k in bwd_names:
                    slot[k].copy_(host_in[k][:, sl], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_copy)
            return slot, ev

        nxt = load_rev(0)
        for i, s in enumerate(order):
            slot, ev = nxt
            if i + 1 < ns:
                nxt = load_rev(i + 1)
            cur.wait_event(ev)
            leaves = [slot["x"].detach().requires_grad_(True), slot["dt"].detach().requires_grad_(True),
                      A_head.detach().requires_grad_(True), slot["B"].detach().requires_grad_(True),
                      slot["C"].detach().requires_grad_(True), D.detach().requires_grad_(True)]
            init = None if states[s] is None else states[s].detach().requires_grad_(True)
            y, final = ssd_mamba2(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], leaves[5], chunk_size, init)
            outs, gouts = [y], [slot["dy"]]
            if dstate is not None:
                outs.append(final)
                gouts.append(dstate)
            ins = leaves + ([init] if init is not None else [])
            grads = torch.autograd.grad(outs, ins, gouts)
            dAh += grads[2].float()
            dD += grads[5].float()
            dstate = grads[6] if init is not None else None
            done = torch.cuda.Event()
            done.record(cur)
            ev_free[i % 2] = done
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                for k, gten in (("dx", grads[0]), ("ddt", grads[1]), ("dB", grads[3]), ("dC", grads[4])):
                    gten.record_stream(self.s_out)
                    host_out[k][:, s * L:(s + 1) * L].copy_(gten, non_blocking=True)
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_out):
            dAh.record_stream(self.s_out)
            dD.record_stream(self.s_out)
            host_out["dA_head"].copy_(dAh, non_blocking=True)
            host_out["dD"].copy_(dD, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_copy)
        self.s_out.synchronize()  # the last copies out are ordered after every kernel: the host may read host_out
