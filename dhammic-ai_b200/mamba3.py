"""Mamba-3 style variant of the scan: data-dependent rotary state angles and the trapezoidal two-term
discretisation.  The reference's block composes it from two scan calls (src/mamba_base_engine.py:137-187):

    gamma = lam * dt                      beta = (1 - lam) * dt * exp(dt * A_head)
    cum   = -cumsum(raw_angles, dim=1)    B_r, C_r = rope(expand(B), cum), rope(expand(C), cum)
    Y = SSD(x * gamma, dt * A_head, B_r, C_r) + SSD(shift(x) * beta, dt * A_head, shift(B_r), C_r) + D * x

The shifted term at position j+1 reaches every later row i with the decay of position j times
``exp(-a[j+1])``, and ``beta[j+1] * exp(-a[j+1]) = (1 - lam[j+1]) * dt[j+1] =: u[j]``; only the row i = j has no
shifted term.  So the same Y is ONE scan with a combined input weight and a diagonal correction:

    w = lam * dt + u          (u[T-1] = 0)           s = <B, C> per group (the rotation preserves it)
    Y = SSD(x * w, dt * A_head, B_r, C_r) + (D - u * s) * x

which halves the scan work and never materialises shift(x) * beta or shift(B_r).  The element-wise steps and
their backward are CUDA kernels of the library (``ssd_b200_m3_prologue_fwd`` / ``_skip_fwd`` / ``_prologue_bwd``);
the scan runs on the scan kernels (one head per group after the per-head rotation).  On the tensor-core path the
scan takes ``w`` and ``D - u * s`` as per-position coefficients (its scaled operator form) and applies them in
its own prologue and epilogue, so ``x * w`` is never written, the skip term costs no pass over y, and the scan's
backward returns the complete ``dx`` together with ``<dX, x>`` and ``<dy, x>``; the fp32 path materialises
``x * w`` and runs the scan in plain operator form.  Unlike
the reference's cached second call (src/kernels/ssd_scan.py:494-500) the decay gradient is the full one of the
expression above; the chain rule on the (b,T,h)-sized tensors (through w, u and a) is one more kernel
(``ssd_b200_m3_chain_bwd``).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _cabi
from .ssd_scan import _dt_code, _ptr, _run_bwd_operator, _run_bwd_scaled, _run_fwd, _stream


def _shape(x: Tensor, B: Tensor) -> _cabi.Shape:
    b, T, h, p = x.shape
    return _cabi.Shape(_cabi.ABI_VERSION, _dt_code(x), _cabi.F32, _cabi.PATH_AUTO, b, T, h, p, B.shape[3], B.shape[2], T)


class _SSDMamba3(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, raw_angles, lam, chunk_size):
        assert x.is_cuda, "ssd_b200 runs on CUDA tensors only (no CPU fallback)"
        lib = _cabi.load()
        chunk = int(chunk_size)
        xc, Bc, Cc = x.contiguous(), B.contiguous(), C_.contiguous()
        # angles keep their own precision: fp32 angles (the reference's dt * theta product) are summed as given
        ang = raw_angles.contiguous() if raw_angles.dtype in (torch.float32, x.dtype) else raw_angles.contiguous().float()
        dtc, lamc, Ah = dt.float().contiguous(), lam.float().contiguous(), A_head.float().contiguous()
        Dc = None if D is None else D.float().contiguous()
        b, T, h, p = xc.shape
        g, n = Bc.shape[2], Bc.shape[3]
        dev = x.device
        shape = _shape(xc, Bc)
        # the scan sees one head per group (per-head rotated B, C)
        scan_probe = _cabi.Shape(_cabi.ABI_VERSION, _dt_code(xc), _cabi.F32, _cabi.PATH_AUTO, b, T, h, p, n, h, chunk)
        fused = lib.ssd_b200_resolve_path(C.byref(scan_probe)) == _cabi.PATH_TC
        with torch.cuda.device(dev):
            dA = torch.empty(b, T, h, dtype=torch.float32, device=dev)
            Br = torch.empty(b, T, h, n, dtype=x.dtype, device=dev)
            Cr = torch.empty_like(Br)
            sdot = torch.empty(b, T, g, dtype=torch.float32, device=dev)
            cum = torch.empty(b, T, h, n // 2, dtype=torch.float32, device=dev)
            seg = torch.empty(b * ((T + 127) // 128) * h * (n // 2), dtype=torch.float32, device=dev)
            xw = None if fused else torch.empty_like(xc)
            w = torch.empty_like(dA) if fused else None
            skip = torch.empty_like(dA) if fused else None
            _cabi.check(lib.ssd_b200_m3_prologue_fwd(C.byref(shape), _ptr(xc), _ptr(dtc), _ptr(lamc), _ptr(Ah), _ptr(Bc),
                                                     _ptr(Cc), _ptr(ang), _dt_code(ang), _ptr(xw), _ptr(dA), _ptr(Br),
                                                     _ptr(Cr), _ptr(sdot), _ptr(cum), _ptr(seg), _ptr(Dc), _ptr(w),
                                                     _ptr(skip), _stream(dev)))
            del seg
            if fused:
                y, final, a_cumsum, scan_shape, states = _run_fwd(xc, dA, w, None, None, Br, Cr, chunk, None, None,
                                                                  want_states=any(ctx.needs_input_grad), skip=skip)
            else:
                y, final, a_cumsum, scan_shape, states = _run_fwd(xw, dA, None, None, None, Br, Cr, chunk, None, None,
                                                                  want_states=any(ctx.needs_input_grad))
                _cabi.check(lib.ssd_b200_m3_skip_fwd(C.byref(shape), _ptr(y), _ptr(xc), _ptr(Dc), _ptr(dtc), _ptr(lamc),
                                                     _ptr(sdot), _ptr(y), _stream(dev)))
        empty = torch.empty(0, device=dev)
        ctx.save_for_backward(xc, dtc, lamc, Ah, Bc, Cc, cum, sdot, xw if xw is not None else empty, dA, Br, Cr, a_cumsum,
                              Dc if Dc is not None else empty, w if fused else empty, skip if fused else empty)
        ctx.states = states
        ctx.fused = fused
        ctx.shape_struct, ctx.scan_shape = shape, scan_shape
        ctx.has_D = D is not None
        ctx.ang_dtype = ang.dtype
        ctx.in_dtypes = (dt.dtype, A_head.dtype, raw_angles.dtype, lam.dtype, None if D is None else D.dtype)
        return y

    @staticmethod
    def backward(ctx, dY):
        x, dt, lam, Ah, B, Cm, cum, sdot, xw, dA, Br, Cr, a_cumsum, D, w, skip = ctx.saved_tensors
        lib = _cabi.load()
        b, T, h, p = x.shape
        g, n = B.shape[2], B.shape[3]
        dev = x.device
        with torch.cuda.device(dev):
            dy = dY.contiguous().to(x.dtype)
            if ctx.fused:  # dx is complete; dw = <dX, x> and dyx = <dy, x> come from the scan's own row sums
                dx, da, dw, dyx, dBr, dCr = _run_bwd_scaled(ctx.scan_shape, x, dA, w, skip, Br, Cr, a_cumsum, dy, ctx.states)
                dxw = None
            else:
                dxw, da, dBr, dCr, _ = _run_bwd_operator(ctx.scan_shape, xw, dA, Br, Cr, a_cumsum, dy, ctx.states)
                dx = torch.empty_like(x)
                dw = torch.empty(b, T, h, dtype=torch.float32, device=dev)
                dyx = torch.empty_like(dw)
            dB, dC = torch.empty_like(B), torch.empty_like(Cm)
            dang = torch.empty(b, T, h, n // 2, dtype=ctx.ang_dtype, device=dev)
            dcum = torch.empty(b, T, h, n // 2, dtype=torch.float32, device=dev)
            seg = torch.empty(b * ((T + 127) // 128) * h * (n // 2), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_m3_prologue_bwd(C.byref(ctx.shape_struct), _ptr(x), _ptr(dy), _ptr(dt), _ptr(lam),
                                                     _ptr(D) if ctx.has_D else None, _ptr(B), _ptr(Cm), _ptr(cum),
                                                     _ptr(sdot), _ptr(dxw), _ptr(dBr), _ptr(dCr), _ptr(dx), _ptr(dw),
                                                     _ptr(dyx), _ptr(dB), _ptr(dC), _ptr(dang), _dt_code(dang), _ptr(dcum),
                                                     _ptr(seg), _stream(dev)))
            # chain rule through w = lam dt + u, u[t] = (1 - lam[t+1]) dt[t+1], the diagonal term -u s x and
            # a = dt A_head, with the two per-head sums, in one kernel on the (b,T,h) tensors
            dlam, ddt = torch.empty_like(dw), torch.empty_like(dw)
            dAh = torch.empty(h, dtype=torch.float32, device=dev)
            dD = torch.empty(h, dtype=torch.float32, device=dev) if ctx.has_D else None
            ws = torch.empty(int(lib.ssd_b200_m3_chain_ws_floats(C.byref(ctx.shape_struct))), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_m3_chain_bwd(C.byref(ctx.shape_struct), _ptr(dw), _ptr(dyx), _ptr(sdot), _ptr(dt),
                                                  _ptr(lam), _ptr(da.contiguous()), _ptr(Ah), _ptr(dlam), _ptr(ddt), _ptr(dAh),
                                                  _ptr(dD), _ptr(ws), _stream(dev)))
        dtd, ahd, angd, lamd, dd = ctx.in_dtypes
        return (dx, ddt.to(dtd), dAh.to(ahd), dB, dC, None if dD is None else dD.to(dd), dang.to(angd), dlam.to(lamd),
                None)


def ssd_mamba3(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor | None, raw_angles: Tensor,
               lam: Tensor, chunk_size: int) -> Tensor:
    """x (b,T,h,p); dt, lam (b,T,h) fp32; A_head, D (h); B, C (b,T,g,n); raw_angles (b,T,h,n/2).  Returns Y."""
    return _SSDMamba3.apply(x, dt, A_head, B, C, D, raw_angles, lam, int(chunk_size))
