"""CPU oracle for the SSD chunked scan -- TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the tests, the smoke
check and the benchmark's CPU-baseline leg may import it.  The shipped
operator must not call anything in here.

It restates, in eager PyTorch on the CPU, the algorithm of the reference's
non-Triton SSD path (paths are relative to the reference's r2/dhammic-ai):

* ``segsum``      -- src/kernels/ssd_scan.py:61-72 (the eager spec quoted
                     there) with the constants of :53-55
* ``exp_clamp``   -- src/kernels/ssd_scan.py:207
* ``ssd_chunked`` -- src/kernels/ssd_scan.py:330-421 (``_ssd_forward_impl``)
* ``fused_ssd_scan_oracle`` -- the wrapper semantics of
                     src/kernels/ssd_scan.py:441-533 and :539-583 (caches are
                     constants in backward, so a cached call yields no decay
                     gradient through them)
* ``ssd_recurrence`` -- the step-by-step recurrence, an independent check
                     (same recurrence as stream/ces/ssd_reference/extract.py:13-63
                     generalised to a head dimension)
* ``mamba2_operator`` -- how the caller forms the scan inputs from x, dt,
                     A_head, D (src/mamba_base_engine.py:170-173, :187 with
                     gamma = dt, i.e. src/kernels/trapezoidal.py:6-12 at lambda = 1)
* ``mamba3_operator`` -- the two-call trapezoidal + rotary composition of
                     src/mamba_base_engine.py:137-187, with the rotation of
                     tests/kernels/test_rope.py:31-43

Parity pinning: ``oracle/pin_against_reference.py`` checks these functions
against the imported reference module (forward, all gradients, the cached
call) and against the reference's 30 stored golden vectors, and writes the
fixtures under tests/golden/.  Status: pinned (see that script's output
recorded in tests/golden/PINNING.txt).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CLAMP_MIN = -20.0
CLAMP_MAX = 20.0
OFF_DIAG_FILL = -1e4


def segsum(x: torch.Tensor) -> torch.Tensor:
    """y[..., i, j] = clamp(sum_{k=j+1..i} x[..., k], -20, 20) for i >= j, clamp(-1e4) above."""
    T = x.shape[-1]
    lower = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
    strict = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device), diagonal=-1)
    xx = x.unsqueeze(-1).expand(*x.shape, T)            # xx[..., i, j] = x[..., i]
    xx = xx.masked_fill(~strict, 0.0)
    s = torch.cumsum(xx, dim=-2)
    s = s + (~lower).to(x.dtype) * OFF_DIAG_FILL
    return s.clamp(CLAMP_MIN, CLAMP_MAX)


def exp_clamp(x: torch.Tensor) -> torch.Tensor:
    return torch.exp(x.clamp(CLAMP_MIN, CLAMP_MAX))


def ssd_chunked(x, A, B, C, chunk_size, initial_states=None,
                L_cache=None, decay_chunk_cache=None, A_cumsum_cache=None):
    """The four-step chunked SSD.  x (b,T,h,p), A (b,T,h), B,C (b,T,h,n).

    Returns (Y (b,T,h,p), final_state (b,h,p,n), {L, decay_chunk, A_cumsum}).
    """
    assert x.shape[1] % chunk_size == 0, (
        f"sequence length {x.shape[1]} not divisible by chunk_size {chunk_size}")
    b, T = x.shape[0], x.shape[1]
    c = T // chunk_size
    xc = x.reshape(b, c, chunk_size, *x.shape[2:])
    Ac = A.reshape(b, c, chunk_size, A.shape[2])
    Bc = B.reshape(b, c, chunk_size, *B.shape[2:])
    Cc = C.reshape(b, c, chunk_size, *C.shape[2:])
    A_perm = Ac.permute(0, 3, 1, 2).contiguous()                     # b h c l
    A_cumsum = A_cumsum_cache if A_cumsum_cache is not None else torch.cumsum(A_perm, dim=-1)
    L = L_cache if L_cache is not None else exp_clamp(segsum(A_perm))
    # step 1: intra-chunk
    Y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", Cc, Bc, L, xc)
    # step 2: per-chunk states
    decay_states = exp_clamp(A_cumsum[:, :, :, -1:] - A_cumsum)
    states = torch.einsum("bclhn,bhcl,bclhp->bchpn", Bc, decay_states, xc)
    # step 3: inter-chunk passing (dense over chunks, as the reference does)
    if initial_states is None:
        initial_states = torch.zeros_like(states[:, :1])
    states_full = torch.cat([initial_states, states], dim=1)
    if decay_chunk_cache is not None:
        decay_chunk = decay_chunk_cache
    else:
        decay_chunk = exp_clamp(segsum(F.pad(A_cumsum[:, :, :, -1], (1, 0))))
    new_states = torch.einsum("bhzc,bchpn->bzhpn", decay_chunk, states_full)
    states_in, final_state = new_states[:, :-1], new_states[:, -1]
    # step 4: state -> output
    Y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", Cc, states_in, exp_clamp(A_cumsum))
    Y = (Y_diag + Y_off).reshape(b, T, x.shape[2], x.shape[3])
    return Y, final_state, {"L": L, "decay_chunk": decay_chunk, "A_cumsum": A_cumsum}


def fused_ssd_scan_oracle(x, A, B, C, chunk_size, initial_states=None, cache=None):
    """Operator-level semantics: a passed cache is trusted and constant in backward."""
    if cache is not None:
        Lc, dc, ac = (cache.get("L"), cache.get("decay_chunk"), cache.get("A_cumsum"))
        Lc = None if Lc is None else Lc.detach()
        dc = None if dc is None else dc.detach()
        ac = None if ac is None else ac.detach()
    else:
        Lc = dc = ac = None
    return ssd_chunked(x, A, B, C, chunk_size, initial_states, Lc, dc, ac)


def ssd_recurrence(x, A, B, C, initial_state=None):
    """H_t = exp(A_t) H_{t-1} + x_t (x) B_t ; y_t = H_t C_t, in float64.  initial_state (b,h,p,n)."""
    x, A, B, C = (t.double() for t in (x, A, B, C))
    b, T, h, p = x.shape
    n = B.shape[-1]
    H = torch.zeros(b, h, p, n, dtype=torch.float64) if initial_state is None else initial_state.double().clone()
    ys = []
    for t in range(T):
        H = torch.exp(A[:, t])[..., None, None] * H + x[:, t, :, :, None] * B[:, t, :, None, :]
        ys.append(torch.einsum("bhpn,bhn->bhp", H, C[:, t]))
    return torch.stack(ys, dim=1), H


def expand_groups(Bg: torch.Tensor, nheads: int) -> torch.Tensor:
    """(b,T,g,n) -> (b,T,h,n): head j uses group j // (h/g)."""
    g = Bg.shape[2]
    assert nheads % g == 0
    return Bg.repeat_interleave(nheads // g, dim=2)


def mamba2_operator(x, dt, A_head, B, C, D, chunk_size, initial_states=None):
    """Y = SSD(x*dt, dt*A_head, B, C) + D*x with B, C given per group."""
    h = x.shape[2]
    Y, final, _ = ssd_chunked(x * dt.unsqueeze(-1), dt * A_head, expand_groups(B, h), expand_groups(C, h),
                              chunk_size, initial_states)
    if D is not None:
        Y = Y + D.view(1, 1, -1, 1) * x
    return Y, final


def apply_rope(v: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotation of the interleaved pairs (v[2m], v[2m+1]) by angles[m], as the reference's eager rotation does
    (tests/kernels/test_rope.py:31-43; kernel src/kernels/rope.py:40-85): even = c x1 - s x2, odd = s x1 + c x2."""
    x1, x2 = v[..., 0::2], v[..., 1::2]
    cs, sn = torch.cos(angles), torch.sin(angles)
    return torch.stack([x1 * cs - x2 * sn, x1 * sn + x2 * cs], dim=-1).flatten(-2)


def trapezoid_coeffs(dt: torch.Tensor, lam: torch.Tensor, A_head: torch.Tensor):
    """(dA, beta, gamma) of the trapezoidal discretisation (src/kernels/trapezoidal.py:6-12;
    tests/kernels/test_trapezoidal.py:20-34 after its softplus / sigmoid / -exp activations)."""
    dA = dt * A_head
    return dA, (1.0 - lam) * dt * torch.exp(dA), lam * dt


def trapezoid_from_raw(dt_raw, lam_raw, dt_bias, A_log):
    """(dt, dA, beta, gamma) from the raw projections, as the reference's eager path does
    (tests/kernels/test_trapezoidal.py:20-34; fused in src/kernels/trapezoidal.py:89-143)."""
    dt = F.softplus(dt_raw + dt_bias)
    lam = torch.sigmoid(lam_raw)
    dA, beta, gamma = trapezoid_coeffs(dt, lam, -torch.exp(A_log))
    return dt, dA, beta, gamma


def mamba3_operator(x, dt, A_head, B, C, D, raw_angles, lam, chunk_size):
    """Two-call trapezoidal composition with data-dependent rotary state angles.

    gamma = lam*dt ; beta = (1-lam)*dt*exp(dt*A_head) ; cum = -cumsum(raw_angles, dim=1);
    Y = SSD(x*gamma, dt*A, rope(B), rope(C)) + SSD(shift(x)*beta, dt*A, shift(rope(B)), rope(C)) + D*x.
    Both calls run under plain autograd (the full decay gradient, unlike the cached operator call).
    """
    h = x.shape[2]
    dA, beta, gamma = trapezoid_coeffs(dt, lam, A_head)
    cum = -torch.cumsum(raw_angles, dim=1)
    Br = apply_rope(expand_groups(B, h), cum)
    Cr = apply_rope(expand_groups(C, h), cum)
    y1, _, _ = ssd_chunked(x * gamma.unsqueeze(-1), dA, Br, Cr, chunk_size)
    B_prev = F.pad(Br[:, :-1], (0, 0, 0, 0, 1, 0))
    x_prev = F.pad(x[:, :-1], (0, 0, 0, 0, 1, 0))
    y2, _, _ = ssd_chunked(x_prev * beta.unsqueeze(-1), dA, B_prev, Cr, chunk_size)
    return y1 + y2 + D.view(1, 1, -1, 1) * x


def mamba2_fwd_bwd(inp: dict, chunk_size: int, dtype=torch.float32, initial_states=None, dfinal=None):
    """Forward + all gradients of the Mamba-2 style operator on (possibly bf16-rounded) inputs,
    evaluated in ``dtype`` on the CPU.  Returns a dict of outputs and gradients."""
    leaf = {k: inp[k].detach().to("cpu").to(dtype).requires_grad_(True) for k in ("x", "dt", "A_head", "B", "C", "D")}
    init = None
    if initial_states is not None:
        init = initial_states.detach().cpu().to(dtype).requires_grad_(True)
    y, final = mamba2_operator(leaf["x"], leaf["dt"], leaf["A_head"], leaf["B"], leaf["C"], leaf["D"],
                               chunk_size, init)
    dy = inp["dy"].detach().cpu().to(dtype)
    outs, gouts = [y], [dy]
    if dfinal is not None:
        outs.append(final)
        gouts.append(dfinal.detach().cpu().to(dtype))
    ins = list(leaf.values()) + ([init] if init is not None else [])
    grads = torch.autograd.grad(outs, ins, gouts)
    res = {"y": y.detach(), "final_state": final.detach()}
    for k, g in zip(list(leaf.keys()) + (["init"] if init is not None else []), grads):
        res["d" + k] = g
    return res


def rel_to_max(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b| -- the parity metric used for every output tensor."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
