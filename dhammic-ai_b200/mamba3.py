"""Mamba-3 style variant of the scan: data-dependent rotary state angles and the trapezoidal two-term
discretisation, composed as the reference's block composes it (src/mamba_base_engine.py:137-187):

    gamma = lam * dt                      beta = (1 - lam) * dt * exp(dt * A_head)
    cum   = -cumsum(raw_angles, dim=1)    B_r, C_r = rope(expand(B), cum), rope(expand(C), cum)
    Y = SSD(x * gamma, dt * A_head, B_r, C_r) + SSD(shift(x) * beta, dt * A_head, shift(B_r), C_r) + D * x

Both scans run on the CUDA kernels of this package (operator form, one head per group after the per-head
rotation).  The element-wise prologue (rotation, products, shifts) is plain tensor arithmetic here, so
autograd carries d raw_angles and d lam; unlike the reference's cached second call
(src/kernels/ssd_scan.py:494-500) both calls contribute to the decay gradient, which is what the full
gradient of the expression above requires.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from .ssd_scan import fused_ssd_scan


def apply_rope(v: Tensor, angles: Tensor) -> Tensor:
    """Pairwise rotation of the two halves of the last dim (tests/kernels/test_rope.py:31-43)."""
    half = v.shape[-1] // 2
    x1, x2 = v[..., :half], v[..., half:]
    cs, sn = torch.cos(angles), torch.sin(angles)
    return torch.cat([x1 * cs - x2 * sn, x1 * sn + x2 * cs], dim=-1)


def ssd_mamba3(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor, raw_angles: Tensor,
               lam: Tensor, chunk_size: int) -> Tensor:
    """x (b,T,h,p); dt, lam (b,T,h) fp32; A_head, D (h); B, C (b,T,g,n); raw_angles (b,T,h,n/2).  Returns Y."""
    h = x.shape[2]
    g = B.shape[2]
    dA = dt.float() * A_head.float()
    gamma = lam.float() * dt.float()
    beta = (1.0 - lam.float()) * dt.float() * torch.exp(dA)
    cum = -torch.cumsum(raw_angles.float(), dim=1)
    Bh = B.float().repeat_interleave(h // g, dim=2)
    Ch = C.float().repeat_interleave(h // g, dim=2)
    Br = apply_rope(Bh, cum).to(x.dtype)
    Cr = apply_rope(Ch, cum).to(x.dtype)
    xg = (x.float() * gamma.unsqueeze(-1)).to(x.dtype)
    y1, _, _ = fused_ssd_scan(xg, dA, Br, Cr, chunk_size)
    B_prev = F.pad(Br[:, :-1], (0, 0, 0, 0, 1, 0))
    x_prev = F.pad(x[:, :-1], (0, 0, 0, 0, 1, 0))
    xb = (x_prev.float() * beta.unsqueeze(-1)).to(x.dtype)
    y2, _, _ = fused_ssd_scan(xb, dA, B_prev, Cr, chunk_size)
    return (y1.float() + y2.float() + D.float().view(1, 1, -1, 1) * x.float()).to(x.dtype)
