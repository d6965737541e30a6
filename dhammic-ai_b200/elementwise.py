"""The element-wise operators around the scan in the reference's block, with the reference's names, argument
order, checks and dtypes, on CUDA kernels of the library:

* ``FusedRoPE`` / ``fused_rope(x, angles)``                                 (src/kernels/rope.py:228-325)
* ``FusedTrapezoidal`` / ``fused_trapezoidal(dt_raw, lam_raw, dt_bias, A_log)``  (src/kernels/trapezoidal.py:220-335)
* ``FusedRMSNorm`` / ``fused_rmsnorm(x, weight, eps)`` / ``FusedRMSNormModule``  (src/kernels/rmsnorm.py:154-245)
* ``fused_gate_norm(y, z, weight, eps)``: the block's closing ``norm(y) * silu(z)``
  (src/mamba_base_engine.py:189-191) in one pass instead of three

Arithmetic is fp32 inside, results are in the input dtype; there is no CPU path (CPU tensors raise, as in the
reference).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from . import _cabi
from .ssd_scan import _dt_code, _ptr, _stream


def _check_rope_inputs(x: Tensor, angles: Tensor):
    assert x.is_cuda and angles.is_cuda, "rotation runs on the GPU only: x and angles must be CUDA tensors"
    assert x.dim() == 4 and angles.dim() == 4, \
        f"x must be (B,T,H,D) and angles (B,T,1 or H,D/2); got {x.dim()} and {angles.dim()} dimensions"
    B, T, H, D = x.shape
    assert D % 2 == 0, f"pairs are rotated, so the last dimension of x must be even (it is {D})"
    aB, aT, aH, aDh = angles.shape
    assert aB == B and aT == T and aDh == D // 2, \
        f"angles {tuple(angles.shape)} do not fit x {tuple(x.shape)}: want ({B}, {T}, 1 or {H}, {D // 2})"
    assert aH == 1 or aH == H, f"angles carry {aH} heads; give 1 (shared by all heads) or {H} (one set per head)"
    return B, T, H, D, aH == 1


class FusedRoPE(torch.autograd.Function):
    """Same call signature as the reference's FusedRoPE (src/kernels/rope.py:228-307)."""

    @staticmethod
    def forward(ctx, x: Tensor, angles: Tensor) -> Tensor:
        B, T, H, D, broadcast_h = _check_rope_inputs(x, angles)
        lib = _cabi.load()
        xc = x.contiguous()
        ang = angles.contiguous().float()
        dev = x.device
        with torch.cuda.device(dev):
            out = torch.empty_like(xc)
            _cabi.check(lib.ssd_b200_rope_fwd(_dt_code(xc), B, T, H, D, int(broadcast_h), _ptr(xc), _ptr(ang), _ptr(out),
                                              _stream(dev)))
        ctx.save_for_backward(xc, ang)
        ctx.dims = (B, T, H, D, broadcast_h)
        ctx.angles_dtype = angles.dtype
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        xc, ang = ctx.saved_tensors
        B, T, H, D, broadcast_h = ctx.dims
        lib = _cabi.load()
        dev = xc.device
        with torch.cuda.device(dev):
            dyc = dy.contiguous().to(xc.dtype)
            dx = torch.empty_like(xc)
            dang = torch.empty(B, T, 1 if broadcast_h else H, D // 2, dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_rope_bwd(_dt_code(xc), B, T, H, D, int(broadcast_h), _ptr(xc), _ptr(ang), _ptr(dyc),
                                              _ptr(dx), _ptr(dang), _stream(dev)))
        return dx, dang.to(ctx.angles_dtype)


def fused_rope(x: Tensor, angles: Tensor) -> Tensor:
    """Rotation of the interleaved pairs of the last dim of x (B,T,H,D) by angles (B,T,1,D/2) or (B,T,H,D/2);
    same contract as the reference (src/kernels/rope.py:310-325)."""
    return FusedRoPE.apply(x, angles)


class FusedTrapezoidal(torch.autograd.Function):
    """Same call signature as the reference's FusedTrapezoidal (src/kernels/trapezoidal.py:220-310)."""

    @staticmethod
    def forward(ctx, dt_raw: Tensor, lam_raw: Tensor, dt_bias: Tensor, A_log: Tensor):
        assert dt_raw.is_cuda and lam_raw.is_cuda and dt_bias.is_cuda and A_log.is_cuda, \
            "the coefficient kernel runs on the GPU only: all four arguments must be CUDA tensors"
        assert dt_raw.shape == lam_raw.shape, \
            f"dt_raw and lam_raw must have one shape, got {tuple(dt_raw.shape)} and {tuple(lam_raw.shape)}"
        assert dt_raw.dim() >= 1, "dt_raw needs a trailing head dimension"
        H = dt_raw.shape[-1]
        assert dt_bias.dim() == 1 and dt_bias.shape[0] == H, f"dt_bias must be ({H},), got {tuple(dt_bias.shape)}"
        assert A_log.dim() == 1 and A_log.shape[0] == H, f"A_log must be ({H},), got {tuple(A_log.shape)}"
        lib = _cabi.load()
        out_dtype = dt_raw.dtype
        dtc = dt_raw.contiguous()
        lamc = lam_raw.contiguous().to(out_dtype)
        # the reference rounds the parameters to the working dtype before use (src/kernels/trapezoidal.py:241-243)
        bias = dt_bias.contiguous().to(out_dtype).float()
        alog = A_log.contiguous().to(out_dtype).float()
        rows = dtc.numel() // H
        dev = dt_raw.device
        with torch.cuda.device(dev):
            dt, dA, beta, gamma = (torch.empty_like(dtc) for _ in range(4))
            _cabi.check(lib.ssd_b200_trapezoid_fwd(_dt_code(dtc), rows, H, _ptr(dtc), _ptr(lamc), _ptr(bias), _ptr(alog),
                                                   _ptr(dt), _ptr(dA), _ptr(beta), _ptr(gamma), _stream(dev)))
        ctx.save_for_backward(dtc, lamc, bias, alog)
        ctx.param_dtypes = (dt_bias.dtype, A_log.dtype)
        return dt, dA, beta, gamma

    @staticmethod
    def backward(ctx, g_dt: Tensor, g_dA: Tensor, g_beta: Tensor, g_gamma: Tensor):
        dtc, lamc, bias, alog = ctx.saved_tensors
        lib = _cabi.load()
        H = dtc.shape[-1]
        rows = dtc.numel() // H
        dev = dtc.device
        with torch.cuda.device(dev):
            gs = [torch.zeros_like(dtc) if g is None else g.contiguous().to(dtc.dtype) for g in (g_dt, g_dA, g_beta, g_gamma)]
            d_dt_raw, d_lam_raw = torch.empty_like(dtc), torch.empty_like(dtc)
            d_bias = torch.empty(H, dtype=torch.float32, device=dev)
            d_alog = torch.empty(H, dtype=torch.float32, device=dev)
            ws = torch.empty(int(lib.ssd_b200_trapezoid_ws_floats(rows, H)), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_trapezoid_bwd(_dt_code(dtc), rows, H, _ptr(dtc), _ptr(lamc), _ptr(bias), _ptr(alog),
                                                   _ptr(gs[0]), _ptr(gs[1]), _ptr(gs[2]), _ptr(gs[3]), _ptr(d_dt_raw),
                                                   _ptr(d_lam_raw), _ptr(d_bias), _ptr(d_alog), _ptr(ws), _stream(dev)))
        bd, ad = ctx.param_dtypes
        return d_dt_raw, d_lam_raw, d_bias.to(bd), d_alog.to(ad)


def fused_trapezoidal(dt_raw: Tensor, lam_raw: Tensor, dt_bias: Tensor, A_log: Tensor):
    """(dt, dA, beta, gamma), each of dt_raw's shape and dtype; same contract as the reference
    (src/kernels/trapezoidal.py:317-335)."""
    return FusedTrapezoidal.apply(dt_raw, lam_raw, dt_bias, A_log)


class FusedRMSNorm(torch.autograd.Function):
    """Same call signature as the reference's FusedRMSNorm (src/kernels/rmsnorm.py:154-219); an optional fourth
    argument z turns it into the gated form ``rmsnorm(x) * silu(z)``."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, eps: float, *gate: Tensor) -> Tensor:
        z = gate[0] if gate else None
        ctx.n_gate = len(gate)
        assert x.is_cuda and weight.is_cuda, "FusedRMSNorm requires CUDA tensors"
        D = x.shape[-1]
        assert weight.dim() == 1 and weight.shape[0] == D, f"weight shape {tuple(weight.shape)} mismatches D={D}"
        if z is not None:
            assert z.is_cuda and z.shape == x.shape, f"gate shape {tuple(z.shape)} vs x {tuple(x.shape)}"
        lib = _cabi.load()
        xc = x.contiguous()
        zc = None if z is None else z.contiguous().to(x.dtype)
        w = weight.contiguous().float()
        rows = xc.numel() // D
        dev = x.device
        with torch.cuda.device(dev):
            out = torch.empty_like(xc)
            rstd = torch.empty(rows, dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_rmsnorm_fwd(_dt_code(xc), rows, D, float(eps), _ptr(xc), _ptr(w), _ptr(zc), _ptr(out),
                                                 _ptr(rstd), _stream(dev)))
        ctx.save_for_backward(xc, w, rstd, zc if zc is not None else torch.empty(0, device=dev))
        ctx.has_gate = z is not None
        ctx.weight_dtype = weight.dtype
        ctx.gate_dtype = None if z is None else z.dtype
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        xc, w, rstd, zc = ctx.saved_tensors
        lib = _cabi.load()
        D = xc.shape[-1]
        rows = xc.numel() // D
        dev = xc.device
        with torch.cuda.device(dev):
            dyc = dy.contiguous().to(xc.dtype)
            dx = torch.empty_like(xc)
            dz = torch.empty_like(xc) if ctx.has_gate else None
            dw = torch.empty(D, dtype=torch.float32, device=dev)
            ws = torch.empty(int(lib.ssd_b200_rmsnorm_ws_floats(rows, D)), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_rmsnorm_bwd(_dt_code(xc), rows, D, _ptr(xc), _ptr(w), _ptr(zc) if ctx.has_gate else None,
                                                 _ptr(dyc), _ptr(rstd), _ptr(dx), _ptr(dz), _ptr(dw), _ptr(ws), _stream(dev)))
        grads = (dx, dw.to(ctx.weight_dtype), None)
        if ctx.n_gate:
            grads += (None if dz is None else dz.to(ctx.gate_dtype),)
        return grads


def fused_rmsnorm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight over the last dim; same contract as the reference
    (src/kernels/rmsnorm.py:222-230)."""
    return FusedRMSNorm.apply(x, weight, eps)


def fused_gate_norm(y: Tensor, z: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """rmsnorm(y, weight, eps) * silu(z), the block's step after the scan (src/mamba_base_engine.py:189-191)."""
    return FusedRMSNorm.apply(y, weight, eps, z)


class FusedRMSNormModule(torch.nn.Module):
    """Same interface as the reference's module (src/kernels/rmsnorm.py:232-245)."""

    def __init__(self, d: int, eps: float = 1e-6):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(d))
        self.eps = eps
        self.d = d

    def forward(self, x: Tensor) -> Tensor:
        return fused_rmsnorm(x, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"d={self.d}, eps={self.eps}"
