"""Mamba-3 style variant of the scan: data-dependent rotary state angles and the trapezoidal two-term
discretisation, composed as the reference's block composes it (src/mamba_base_engine.py:137-187):

    gamma = lam * dt                      beta = (1 - lam) * dt * exp(dt * A_head)
    cum   = -cumsum(raw_angles, dim=1)    B_r, C_r = rope(expand(B), cum), rope(expand(C), cum)
    Y = SSD(x * gamma, dt * A_head, B_r, C_r) + SSD(shift(x) * beta, dt * A_head, shift(B_r), C_r) + D * x

The element-wise prologue (angle scan, rotation, products, shifts) and its backward are CUDA kernels of the
library (``ssd_b200_m3_prologue_fwd`` / ``_bwd``); both scans run on the scan kernels in operator form (one
head per group after the per-head rotation).  Unlike the reference's cached second call
(src/kernels/ssd_scan.py:494-500) both calls contribute to the decay gradient, which is what the full
gradient of the expression above requires.  Only arithmetic on (b,T,h)-sized tensors (the chain rule through
gamma and beta) and the final ``y1 + y2 + D x`` are left to tensor operations.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _cabi
from .ssd_scan import _dt_code, _ptr, _stream, fused_ssd_scan


def _shape(x: Tensor, B: Tensor) -> _cabi.Shape:
    b, T, h, p = x.shape
    return _cabi.Shape(_cabi.ABI_VERSION, _dt_code(x), _cabi.F32, _cabi.PATH_AUTO, b, T, h, p, B.shape[3], B.shape[2], T)


class _M3Prologue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, raw_angles, lam):
        assert x.is_cuda, "ssd_b200 runs on CUDA tensors only (no CPU fallback)"
        lib = _cabi.load()
        xc, Bc, Cc = x.contiguous(), B.contiguous(), C_.contiguous()
        ang = raw_angles.contiguous().to(x.dtype)
        dtc, lamc, Ah = dt.float().contiguous(), lam.float().contiguous(), A_head.float().contiguous()
        b, T, h, p = xc.shape
        n = Bc.shape[3]
        dev = x.device
        shape = _shape(xc, Bc)
        with torch.cuda.device(dev):
            xg, xb = torch.empty_like(xc), torch.empty_like(xc)
            dA = torch.empty(b, T, h, dtype=torch.float32, device=dev)
            Br = torch.empty(b, T, h, n, dtype=x.dtype, device=dev)
            Cr, Bprev = torch.empty_like(Br), torch.empty_like(Br)
            cum = torch.empty(b, T, h, n // 2, dtype=torch.float32, device=dev)
            seg = torch.empty(b * ((T + 127) // 128) * h * (n // 2), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_m3_prologue_fwd(C.byref(shape), _ptr(xc), _ptr(dtc), _ptr(lamc), _ptr(Ah), _ptr(Bc),
                                                     _ptr(Cc), _ptr(ang), _ptr(xg), _ptr(xb), _ptr(dA), _ptr(Br), _ptr(Cr),
                                                     _ptr(Bprev), _ptr(cum), _ptr(seg), _stream(dev)))
        ctx.save_for_backward(xc, dtc, lamc, Ah, Bc, Cc, cum, dA)
        ctx.shape_struct = shape
        ctx.in_dtypes = (dt.dtype, A_head.dtype, raw_angles.dtype, lam.dtype)
        return xg, xb, dA, Br, Cr, Bprev

    @staticmethod
    def backward(ctx, dxg, dxb, ddA, dBr, dCr, dBprev):
        x, dt, lam, Ah, B, Cm, cum, dA = ctx.saved_tensors
        lib = _cabi.load()
        b, T, h, p = x.shape
        n = B.shape[3]
        dev = x.device
        with torch.cuda.device(dev):
            def full(g, shape):
                return torch.zeros(shape, dtype=x.dtype, device=dev) if g is None else g.contiguous().to(x.dtype)
            dxg, dxb = full(dxg, x.shape), full(dxb, x.shape)
            dBr, dCr, dBprev = full(dBr, (b, T, h, n)), full(dCr, (b, T, h, n)), full(dBprev, (b, T, h, n))
            zero_r = torch.zeros_like(dCr)
            zero_x = torch.zeros_like(x)  # the D skip and its gradient stay outside this function
            dx = torch.empty_like(x)
            dgam = torch.empty(b, T, h, dtype=torch.float32, device=dev)
            dbet, dyx = torch.empty_like(dgam), torch.empty_like(dgam)
            dB, dC = torch.empty_like(B), torch.empty_like(Cm)
            dang = torch.empty(b, T, h, n // 2, dtype=x.dtype, device=dev)
            dcum = torch.empty(b, T, h, n // 2, dtype=torch.float32, device=dev)
            seg = torch.empty(b * ((T + 127) // 128) * h * (n // 2), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_m3_prologue_bwd(C.byref(ctx.shape_struct), _ptr(x), _ptr(zero_x), _ptr(dt), _ptr(lam),
                                                     _ptr(Ah), None, _ptr(B), _ptr(Cm), _ptr(cum), _ptr(dxg), _ptr(dxb),
                                                     _ptr(dBr), _ptr(dBprev), _ptr(dCr), _ptr(zero_r), _ptr(dx), _ptr(dgam),
                                                     _ptr(dbet), _ptr(dyx), _ptr(dB), _ptr(dC), _ptr(dang), _ptr(dcum),
                                                     _ptr(seg), _stream(dev)))
            # chain rule through gamma = lam dt, beta = (1 - lam) dt exp(a), a = dt A_head   [(b,T,h)-sized]
            ea = torch.exp(dA)
            beta = (1.0 - lam) * dt * ea
            da_tot = dbet * beta if ddA is None else ddA.float() + dbet * beta
            dlam = dgam * dt - dbet * dt * ea
            ddt = dgam * lam + dbet * (1.0 - lam) * ea + da_tot * Ah
            dAh = (da_tot * dt).sum(dim=(0, 1))
        dtd, ahd, angd, lamd = ctx.in_dtypes
        return dx, ddt.to(dtd), dAh.to(ahd), dB, dC, dang.to(angd), dlam.to(lamd)


def ssd_mamba3(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor, raw_angles: Tensor,
               lam: Tensor, chunk_size: int) -> Tensor:
    """x (b,T,h,p); dt, lam (b,T,h) fp32; A_head, D (h); B, C (b,T,g,n); raw_angles (b,T,h,n/2).  Returns Y."""
    xg, xb, dA, Br, Cr, Bprev = _M3Prologue.apply(x, dt, A_head, B, C, raw_angles, lam)
    y1, _, _ = fused_ssd_scan(xg, dA, Br, Cr, chunk_size)
    y2, _, _ = fused_ssd_scan(xb, dA, Bprev, Cr, chunk_size)
    return torch.addcmul(y1 + y2, x, D.to(x.dtype).view(1, 1, -1, 1))
