"""Host side of the B200 SSD chunked scan: the reference's operator interface over the C ABI.

``FusedSSDScan`` and ``fused_ssd_scan`` keep the names, argument order, return
arity, cache keys and error behaviour of the reference operator
(src/kernels/ssd_scan.py:427-465, :468-533, :539-583) so that the only
production caller (src/mamba_base_engine.py:170-181) runs unchanged.  All
arithmetic happens in the CUDA library behind include/ssd_b200.h; PyTorch here
only owns device memory and the stream.  There is no CPU or eager fallback:
non-CUDA tensors raise, as in the reference (src/kernels/ssd_scan.py:247).

Differences from the reference, all deliberate:

* ``A`` may be fp32 while x/B/C are bf16; the chunk cumsum, decay factors,
  states and accumulators are always fp32 (the reference keeps them in the
  input dtype).  ``cache["A_cumsum"]`` is therefore fp32.
* ``B``/``C`` may have fewer heads than ``x`` (groups): (b,T,g,n) with g | h.
* ``L`` and ``decay_chunk`` are not needed by these kernels.  The returned
  cache materialises them on first access (same shapes and values as the
  reference, tests/kernels/test_ssd_scan.py:107-110); ``set_eager_cache(True)``
  makes ``FusedSSDScan.apply`` return them eagerly instead of ``None``.
* Backward is a closed form (no re-run under autograd, no host sync such as
  the reference's ``dfinal_state.abs().sum() > 0``, src/kernels/ssd_scan.py:506).
* A cached call returns no gradient for ``A``, exactly like the reference
  (src/kernels/ssd_scan.py:494-500, :533).

``ssd_mamba2`` is the same scan with the caller's input products fused:
Y = SSD(x*dt, dt*A_head, B, C) + D*x with gradients dx, ddt, dA_head, dB, dC, dD.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
from torch import Tensor

from . import _cabi

_EAGER_CACHE = False
_FORCE_PATH = _cabi.PATH_AUTO
_CHECK_STATUS = os.environ.get("SSD_B200_CHECK_STATUS", "0") == "1"
_SAVE_STATES = os.environ.get("SSD_B200_SAVE_STATES", "1") == "1"


def set_save_states(flag: bool) -> None:
    """Keep the per-tile recurrent states of the forward for the backward (default on: one bf16 buffer of
    b*T*h*64 elements, the size of x at d_state 128) instead of recomputing them in the backward, which is
    what the reference's input-only checkpointing corresponds to (src/kernels/ssd_scan.py:458)."""
    global _SAVE_STATES
    _SAVE_STATES = bool(flag)


def set_check_status(flag: bool) -> None:
    """After every call, synchronise and raise if a kernel reported a bounded wait that ran out
    (debug / test use: it costs a stream synchronisation per call)."""
    global _CHECK_STATUS
    _CHECK_STATUS = bool(flag)


def _status(lib, shape, ws, dev) -> None:
    if _CHECK_STATUS:
        _cabi.check(lib.ssd_b200_device_status(C.byref(shape), _ptr(ws), _stream(dev)))


def set_eager_cache(flag: bool) -> None:
    """Make FusedSSDScan.apply return materialised L / decay_chunk tensors (default: None, lazy)."""
    global _EAGER_CACHE
    _EAGER_CACHE = bool(flag)


def set_kernel_path(path: str) -> None:
    """'auto' (default), 'simt' (fp32 SIMT kernels) or 'tc' (tcgen05 kernels; raises if unsupported)."""
    global _FORCE_PATH
    _FORCE_PATH = {"auto": _cabi.PATH_AUTO, "simt": _cabi.PATH_SIMT, "tc": _cabi.PATH_TC}[path]


def _dt_code(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return _cabi.F32
    if t.dtype == torch.bfloat16:
        return _cabi.BF16
    raise RuntimeError(f"ssd_b200 supports float32 and bfloat16 tensors, got {t.dtype}")


def _ptr(t: Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(dev) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _make_shape(x: Tensor, a_dtype: int, B: Tensor, chunk: int) -> _cabi.Shape:
    b, T, h, p = x.shape
    return _cabi.Shape(_cabi.ABI_VERSION, _dt_code(x), a_dtype, _FORCE_PATH, b, T, h, p, B.shape[3], B.shape[2],
                       int(chunk))


def _workspace(lib, shape: _cabi.Shape, which: int, dev) -> Tensor:
    nbytes = lib.ssd_b200_workspace_bytes(C.byref(shape), which)
    if nbytes == 0:
        _cabi.check(lib.ssd_b200_resolve_path(C.byref(shape)))
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)


def _check_inputs(x: Tensor, B: Tensor, Cm: Tensor) -> None:
    assert x.is_cuda and B.is_cuda and Cm.is_cuda, "ssd_b200 runs on CUDA tensors only (no CPU fallback)"
    if x.dim() != 4 or B.dim() != 4 or Cm.dim() != 4:
        raise ValueError("expected x (b,T,h,p) and B, C (b,T,g,n)")
    if B.shape != Cm.shape or B.shape[:2] != x.shape[:2]:
        raise ValueError(f"shape mismatch: x {tuple(x.shape)}, B {tuple(B.shape)}, C {tuple(Cm.shape)}")
    if not (x.dtype == B.dtype == Cm.dtype):
        raise RuntimeError(f"expected x, B and C to have the same dtype, got {x.dtype}, {B.dtype}, {Cm.dtype}")


class LazySSDCache(dict):
    """The operator's cache dict.  ``A_cumsum`` is always present; ``L`` and ``decay_chunk`` are built
    by a small kernel the first time they are read (the production caller only hands the dict back)."""

    def __init__(self, a_cumsum: Tensor, shape: _cabi.Shape, out_dtype: torch.dtype):
        super().__init__(A_cumsum=a_cumsum)
        self._shape = shape
        self._dtype = out_dtype

    def _materialize(self, key: str) -> Tensor:
        s = self._shape
        cum = dict.__getitem__(self, "A_cumsum")
        c = s.seqlen // s.chunk
        with torch.cuda.device(cum.device):
            if key == "L":
                out = torch.empty(s.batch, s.nheads, c, s.chunk, s.chunk, dtype=self._dtype, device=cum.device)
                args = (_ptr(out), None)
            else:
                out = torch.empty(s.batch, s.nheads, c + 1, c + 1, dtype=self._dtype, device=cum.device)
                args = (None, _ptr(out))
            lib = _cabi.load()
            _cabi.check(lib.ssd_b200_materialize_cache(C.byref(s), _ptr(cum), args[0], args[1], _dt_code(out),
                                                       _stream(cum.device)))
        dict.__setitem__(self, key, out)
        return out

    def __missing__(self, key):
        if key in ("L", "decay_chunk"):
            return self._materialize(key)
        raise KeyError(key)

    def get(self, key, default=None):
        if key in ("L", "decay_chunk", "A_cumsum"):
            return self[key]
        return dict.get(self, key, default)

    def __contains__(self, key):
        return key in ("L", "decay_chunk", "A_cumsum") or dict.__contains__(self, key)

    def keys(self):
        return ["L", "decay_chunk", "A_cumsum"]

    def peek(self, key):
        """Read an entry without materialising it (None if not built yet)."""
        return dict.get(self, key)


def _run_fwd(x, a, dt, A_head, D, B, Cm, chunk, init4, a_cumsum_in, want_states=False, ysq=None, skip=None, states=None,
             aux_valid=False):
    """Common forward launcher.  Returns (y, final_state fp32 (b,h,p,n), a_cumsum, shape, states or None).
    ``ysq``: optional fp32 buffer (b, T/128, h, 2, 128) for the per-half-row sums of y^2 (tensor-core path).
    ``states``: a buffer to use instead of allocating one; with ``aux_valid`` its per-position arrays were filled by an
    earlier call on the same inputs and are reused."""
    lib = _cabi.load()
    b, T, h, p = x.shape
    n = B.shape[3]
    dev = x.device
    assert T % chunk == 0, f"sequence length {T} not divisible by chunk_size {chunk}"
    a_dtype = _dt_code(a) if a is not None else _cabi.F32
    shape = _make_shape(x, a_dtype, B, chunk)
    with torch.cuda.device(dev):
        y = torch.empty_like(x)
        final = torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
        if a_cumsum_in is not None:
            cum = a_cumsum_in
            if cum.dtype != torch.float32 or not cum.is_contiguous():
                cum = cum.float().contiguous()
            if tuple(cum.shape) != (b, h, T // chunk, chunk):
                raise ValueError(f"A_cumsum cache has shape {tuple(cum.shape)}, expected {(b, h, T // chunk, chunk)}")
        else:
            cum = torch.empty(b, h, T // chunk, chunk, dtype=torch.float32, device=dev)
        ws = _workspace(lib, shape, _cabi.PASS_FWD, dev)
        if states is None and want_states and _SAVE_STATES:
            nbytes = lib.ssd_b200_states_bytes(C.byref(shape))
            if nbytes:
                states = torch.empty(int(nbytes), dtype=torch.uint8, device=dev)
        flags = _cabi.FWD_AUX_VALID if (aux_valid and states is not None) else 0
        args = _cabi.FwdArgs(shape, _ptr(x), _ptr(a), _ptr(dt), _ptr(A_head), _ptr(D), _ptr(B), _ptr(Cm), _ptr(init4),
                             _ptr(y), _ptr(final), _ptr(cum), 1 if a_cumsum_in is not None else 0, flags, _ptr(ws),
                             ws.numel(), _ptr(states), None, _ptr(ysq), _ptr(skip))
        _cabi.check(lib.ssd_b200_fwd(C.byref(args), _stream(dev)))
        _status(lib, shape, ws, dev)
    return y, final, cum, shape, states


def _run_bwd_operator(shape, x, A, B, Cm, cum, dY, states, init4=None, dfinal_state=None, cached=False):
    """Backward launcher of the operator form (log-decay A given per position).  Returns
    (dx, dA fp32 (b,T,h) or None when ``cached``, dB, dC, d initial state fp32 or None)."""
    lib = _cabi.load()
    dev = x.device
    b, T, h, p = x.shape
    with torch.cuda.device(dev):
        dy = dY.contiguous()
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        dfin = None if dfinal_state is None else dfinal_state.float().contiguous()
        dx = torch.empty_like(x)
        dB = torch.empty_like(B)
        dC = torch.empty_like(Cm)
        da = None if cached else torch.empty(b, T, h, dtype=torch.float32, device=dev)
        dinit = torch.empty(b, h, p, B.shape[3], dtype=torch.float32, device=dev) if init4 is not None else None
        ws = _workspace(lib, shape, _cabi.PASS_BWD, dev)
        args = _cabi.BwdArgs(shape, _ptr(x), _ptr(A), None, None, None, _ptr(B), _ptr(Cm), _ptr(init4), _ptr(cum),
                             _ptr(dy), _ptr(dfin), _ptr(dx), _ptr(dB), _ptr(dC), _ptr(da), None, None, None, _ptr(dinit),
                             1 if cached else 0, 0, _ptr(ws), ws.numel(), _ptr(states))
        _cabi.check(lib.ssd_b200_bwd(C.byref(args), _stream(dev)))
        _status(lib, shape, ws, dev)
    return dx, da, dB, dC, dinit


class FusedSSDScan(torch.autograd.Function):
    """Same call signature as the reference's FusedSSDScan (src/kernels/ssd_scan.py:441-465)."""

    @staticmethod
    def forward(ctx, x: Tensor, A: Tensor, B: Tensor, C_: Tensor, chunk_size: int,
                initial_states: Tensor | None, L_cache_in: Tensor | None,
                decay_chunk_cache_in: Tensor | None, A_cumsum_cache_in: Tensor | None):
        ctx.set_materialize_grads(False)  # an unused final state must not cost a zero tensor and a seeded reverse walk
        _check_inputs(x, B, C_)
        assert A.is_cuda
        chunk = int(chunk_size)
        xc, Ac, Bc, Cc = x.contiguous(), A.contiguous(), B.contiguous(), C_.contiguous()
        b, T, h, p = xc.shape
        n = Bc.shape[3]
        init4 = None
        if initial_states is not None:
            init4 = initial_states.reshape(b, h, p, n).float().contiguous()
        cached = A_cumsum_cache_in is not None
        y, final, cum, shape, states = _run_fwd(xc, Ac, None, None, None, Bc, Cc, chunk, init4,
                                                A_cumsum_cache_in if cached else None,
                                                want_states=any(ctx.needs_input_grad))
        ctx.states = states
        ctx.save_for_backward(xc, Ac, Bc, Cc, init4 if init4 is not None else torch.empty(0, device=x.device), cum)
        ctx.chunk = chunk
        ctx.has_init = initial_states is not None
        ctx.init_shape = None if initial_states is None else tuple(initial_states.shape)
        ctx.init_dtype = None if initial_states is None else initial_states.dtype
        ctx.cached = cached
        ctx.shape_struct = shape
        ctx.mark_non_differentiable(cum)
        L = dc = None
        if _EAGER_CACHE:
            lazy = LazySSDCache(cum, shape, x.dtype)
            L = L_cache_in.detach() if L_cache_in is not None else lazy["L"]
            dc = decay_chunk_cache_in.detach() if decay_chunk_cache_in is not None else lazy["decay_chunk"]
            ctx.mark_non_differentiable(L, dc)
        return y, final.to(x.dtype), L, dc, cum

    @staticmethod
    def backward(ctx, dY, dfinal_state, dL_unused, ddecay_chunk_unused, dA_cumsum_unused):
        x, A, B, Cm, init4, cum = ctx.saved_tensors
        if dY is None:
            dY = torch.zeros_like(x)
        dx, da, dB, dC, dinit = _run_bwd_operator(ctx.shape_struct, x, A, B, Cm, cum, dY, ctx.states,
                                                  init4 if ctx.has_init else None, dfinal_state, ctx.cached)
        dA = None if da is None else da.to(A.dtype)
        dis = None
        if ctx.has_init:
            dis = dinit.reshape(ctx.init_shape).to(ctx.init_dtype)
        return dx, dA, dB, dC, None, dis, None, None, None


def fused_ssd_scan(x: Tensor, A: Tensor, B: Tensor, C: Tensor, chunk_size: int,
                   initial_states: Tensor | None = None, cache: dict | None = None):
    """Fused SSD chunked scan; same contract as the reference (src/kernels/ssd_scan.py:539-583).

    x (b,T,h,p); A (b,T,h) log-decay; B, C (b,T,h,n) (or (b,T,g,n)); initial_states (b,1,h,p,n).
    Returns (Y (b,T,h,p), final_state (b,h,p,n), cache {L, decay_chunk, A_cumsum}).
    """
    if cache is not None:
        if isinstance(cache, LazySSDCache):
            L_in, dc_in, ac_in = cache.peek("L"), cache.peek("decay_chunk"), cache.peek("A_cumsum")
        else:
            L_in, dc_in, ac_in = cache.get("L"), cache.get("decay_chunk"), cache.get("A_cumsum")
            if ac_in is None and (L_in is not None or dc_in is not None):
                raise ValueError("a cache must carry A_cumsum; L and decay_chunk alone cannot be reused here")
    else:
        L_in = dc_in = ac_in = None
    Y, final_state, L_out, dc_out, ac_out = FusedSSDScan.apply(
        x, A, B, C, int(chunk_size), initial_states, L_in, dc_in, ac_in)
    out_cache = LazySSDCache(ac_out, _make_shape(x, _cabi.F32, B, int(chunk_size)), x.dtype)
    for k, v in (("L", L_out if L_out is not None else L_in), ("decay_chunk", dc_out if dc_out is not None else dc_in)):
        if v is not None:
            dict.__setitem__(out_cache, k, v)
    return Y, final_state, out_cache


class _SSDMamba2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, chunk_size, initial_states):
        _check_inputs(x, B, C_)
        ctx.set_materialize_grads(False)  # an unused final state must not cost a zero tensor and a seeded reverse walk
        chunk = int(chunk_size)
        xc, Bc, Cc = x.contiguous(), B.contiguous(), C_.contiguous()
        dtc = dt.float().contiguous()
        Ah = A_head.float().contiguous()
        Dc = None if D is None else D.float().contiguous()
        b, T, h, p = xc.shape
        n = Bc.shape[3]
        init4 = None if initial_states is None else initial_states.reshape(b, h, p, n).float().contiguous()
        y, final, cum, shape, states = _run_fwd(xc, None, dtc, Ah, Dc, Bc, Cc, chunk, init4, None,
                                                want_states=any(ctx.needs_input_grad))
        ctx.states = states
        ctx.save_for_backward(xc, dtc, Ah, Bc, Cc, cum,
                              Dc if Dc is not None else torch.empty(0, device=x.device),
                              init4 if init4 is not None else torch.empty(0, device=x.device))
        ctx.has_D = D is not None
        ctx.has_init = initial_states is not None
        ctx.init_shape = None if initial_states is None else tuple(initial_states.shape)
        ctx.shape_struct = shape
        ctx.in_dtypes = (dt.dtype, A_head.dtype, None if D is None else D.dtype)
        return y, final

    @staticmethod
    def backward(ctx, dY, dfinal):
        x, dt, Ah, B, Cm, cum, D, init4 = ctx.saved_tensors
        if dY is None:
            dY = torch.zeros_like(x)
        lib = _cabi.load()
        shape = ctx.shape_struct
        dev = x.device
        b, T, h, p = x.shape
        with torch.cuda.device(dev):
            dy = dY.contiguous().to(x.dtype)
            dfin = None if dfinal is None else dfinal.float().contiguous()
            dx = torch.empty_like(x)
            dB = torch.empty_like(B)
            dC = torch.empty_like(Cm)
            ddt = torch.empty(b, T, h, dtype=torch.float32, device=dev)
            dAh = torch.empty(h, dtype=torch.float32, device=dev)
            dD = torch.empty(h, dtype=torch.float32, device=dev) if ctx.has_D else None
            dinit = torch.empty(b, h, p, B.shape[3], dtype=torch.float32, device=dev) if ctx.has_init else None
            ws = _workspace(lib, shape, _cabi.PASS_BWD, dev)
            args = _cabi.BwdArgs(shape, _ptr(x), None, _ptr(dt), _ptr(Ah), _ptr(D) if ctx.has_D else None, _ptr(B),
                                 _ptr(Cm), _ptr(init4) if ctx.has_init else None, _ptr(cum), _ptr(dy), _ptr(dfin),
                                 _ptr(dx), _ptr(dB), _ptr(dC), None, _ptr(ddt), _ptr(dAh), _ptr(dD), _ptr(dinit),
                                 0, 0, _ptr(ws), ws.numel(), _ptr(ctx.states))
            _cabi.check(lib.ssd_b200_bwd(C.byref(args), _stream(dev)))
            _status(lib, shape, ws, dev)
        dtd, ahd, dd = ctx.in_dtypes
        return (dx, ddt.to(dtd), dAh.to(ahd), dB, dC, None if dD is None else dD.to(dd), None,
                None if dinit is None else dinit.reshape(ctx.init_shape))


def ssd_mamba2(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor | None, chunk_size: int,
               initial_states: Tensor | None = None):
    """Y = SSD(x*dt, dt*A_head, B, C) + D*x, the scan as the caller composes it
    (src/mamba_base_engine.py:170-173, :187 with gamma = dt), in one call.

    x (b,T,h,p) bf16/fp32; dt (b,T,h); A_head (h); B, C (b,T,g,n); D (h) or None;
    initial_states (b,h,p,n) or (b,1,h,p,n).  Returns (Y, final_state fp32 (b,h,p,n)).
    """
    return _SSDMamba2.apply(x, dt, A_head, B, C, D, int(chunk_size), initial_states)


def _run_bwd_scaled(shape, x, a, w, skip, B, Cm, cum, dY, states):
    """Backward launcher of the scaled operator form (X = x * w, log-decay a, y += skip * x).  Returns
    (dx, da, dw, dskip, dB, dC): dx complete, the three (b,T,h) gradients fp32."""
    lib = _cabi.load()
    dev = x.device
    b, T, h, p = x.shape
    with torch.cuda.device(dev):
        dy = dY.contiguous().to(x.dtype)
        dx, dB, dC = torch.empty_like(x), torch.empty_like(B), torch.empty_like(Cm)
        da = torch.empty(b, T, h, dtype=torch.float32, device=dev)
        dw, dskip = torch.empty_like(da), torch.empty_like(da)
        ws = _workspace(lib, shape, _cabi.PASS_BWD, dev)
        args = _cabi.BwdArgs(shape, _ptr(x), _ptr(a), _ptr(w), None, None, _ptr(B), _ptr(Cm), None, _ptr(cum), _ptr(dy),
                             None, _ptr(dx), _ptr(dB), _ptr(dC), _ptr(da), _ptr(dw), None, None, None, 0, 0, _ptr(ws),
                             ws.numel(), _ptr(states), _ptr(skip), _ptr(dskip))
        _cabi.check(lib.ssd_b200_bwd(C.byref(args), _stream(dev)))
        _status(lib, shape, ws, dev)
    return dx, da, dw, dskip, dB, dC


def _mamba2_backward(ctx_shape, x, dt, Ah, B, Cm, cum, D, init4, states, dY, dfinal, has_D, has_init):
    """Backward launcher of the Mamba-2 form; returns (dx, ddt, dA_head, dB, dC, dD or None, dinit or None), fp32
    for the small ones."""
    lib = _cabi.load()
    dev = x.device
    b, T, h, p = x.shape
    with torch.cuda.device(dev):
        dy = dY.contiguous().to(x.dtype)
        dfin = None if dfinal is None else dfinal.float().contiguous()
        dx = torch.empty_like(x)
        dB = torch.empty_like(B)
        dC = torch.empty_like(Cm)
        ddt = torch.empty(b, T, h, dtype=torch.float32, device=dev)
        dAh = torch.empty(h, dtype=torch.float32, device=dev)
        dD = torch.empty(h, dtype=torch.float32, device=dev) if has_D else None
        dinit = torch.empty(b, h, p, B.shape[3], dtype=torch.float32, device=dev) if has_init else None
        ws = _workspace(lib, ctx_shape, _cabi.PASS_BWD, dev)
        args = _cabi.BwdArgs(ctx_shape, _ptr(x), None, _ptr(dt), _ptr(Ah), _ptr(D) if has_D else None, _ptr(B),
                             _ptr(Cm), _ptr(init4) if has_init else None, _ptr(cum), _ptr(dy), _ptr(dfin),
                             _ptr(dx), _ptr(dB), _ptr(dC), None, _ptr(ddt), _ptr(dAh), _ptr(dD), _ptr(dinit),
                             0, 0, _ptr(ws), ws.numel(), _ptr(states))
        _cabi.check(lib.ssd_b200_bwd(C.byref(args), _stream(dev)))
        _status(lib, ctx_shape, ws, dev)
    return dx, ddt, dAh, dB, dC, dD, dinit


class _SSDMamba2Gated(torch.autograd.Function):
    """The scan followed by the block's output stage, out = rmsnorm(y over all heads) * silu(z)
    (src/mamba_base_engine.py:189-191), as one operator.  The forward walk leaves the per-half-row sums of y^2
    behind, so the norm reads y once; y itself is kept (the norm's backward needs it)."""

    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, z, norm_weight, eps, chunk_size, initial_states):
        _check_inputs(x, B, C_)
        ctx.set_materialize_grads(False)
        lib = _cabi.load()
        chunk = int(chunk_size)
        xc, Bc, Cc = x.contiguous(), B.contiguous(), C_.contiguous()
        dtc = dt.float().contiguous()
        Ah = A_head.float().contiguous()
        Dc = None if D is None else D.float().contiguous()
        b, T, h, p = xc.shape
        n = Bc.shape[3]
        dev = x.device
        assert z.is_cuda and z.shape[:2] == x.shape[:2] and z.numel() == x.numel(), \
            f"the gate must have the size of y: {tuple(z.shape)} vs {tuple(x.shape)}"
        init4 = None if initial_states is None else initial_states.reshape(b, h, p, n).float().contiguous()
        shape = _make_shape(xc, _cabi.F32, Bc, chunk)
        path = lib.ssd_b200_resolve_path(C.byref(shape))
        _cabi.check(path)
        with torch.cuda.device(dev):
            ysq = None
            if path == _cabi.PATH_TC:
                ysq = torch.empty(b * (T // 128) * h * 2 * 128, dtype=torch.float32, device=dev)
            y, final, cum, shape, states = _run_fwd(xc, None, dtc, Ah, Dc, Bc, Cc, chunk, init4, None,
                                                    want_states=any(ctx.needs_input_grad), ysq=ysq)
            zc = z.contiguous().to(xc.dtype).reshape(b * T, h * p)
            w = norm_weight.contiguous().float()
            out = torch.empty_like(y)
            rstd = torch.empty(b * T, dtype=torch.float32, device=dev)
            if ysq is not None:
                _cabi.check(lib.ssd_b200_rmsnorm_fwd_presummed(_dt_code(y), b * T, h * p, float(eps), _ptr(y), _ptr(w),
                                                               _ptr(zc), _ptr(ysq), h, _ptr(out), _ptr(rstd), _stream(dev)))
            else:
                _cabi.check(lib.ssd_b200_rmsnorm_fwd(_dt_code(y), b * T, h * p, float(eps), _ptr(y), _ptr(w), _ptr(zc),
                                                     _ptr(out), _ptr(rstd), _stream(dev)))
        ctx.states = states
        ctx.save_for_backward(xc, dtc, Ah, Bc, Cc, cum,
                              Dc if Dc is not None else torch.empty(0, device=dev),
                              init4 if init4 is not None else torch.empty(0, device=dev), y, zc, w, rstd)
        ctx.has_D = D is not None
        ctx.has_init = initial_states is not None
        ctx.init_shape = None if initial_states is None else tuple(initial_states.shape)
        ctx.shape_struct = shape
        ctx.in_dtypes = (dt.dtype, A_head.dtype, None if D is None else D.dtype, z.dtype, norm_weight.dtype)
        ctx.z_shape = tuple(z.shape)
        return out, final

    @staticmethod
    def backward(ctx, dout, dfinal):
        x, dt, Ah, B, Cm, cum, D, init4, y, zc, w, rstd = ctx.saved_tensors
        if dout is None:
            dout = torch.zeros_like(x)
        lib = _cabi.load()
        dev = x.device
        b, T, h, p = x.shape
        rows, Dn = b * T, h * p
        with torch.cuda.device(dev):
            do = dout.contiguous().to(x.dtype).reshape(rows, Dn)
            dy = torch.empty_like(y)
            dz = torch.empty_like(zc)
            dw = torch.empty(Dn, dtype=torch.float32, device=dev)
            ws = torch.empty(int(lib.ssd_b200_rmsnorm_ws_floats(rows, Dn)), dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_rmsnorm_bwd(_dt_code(y), rows, Dn, _ptr(y), _ptr(w), _ptr(zc), _ptr(do), _ptr(rstd),
                                                 _ptr(dy), _ptr(dz), _ptr(dw), _ptr(ws), _stream(dev)))
        dx, ddt, dAh, dB, dC, dD, dinit = _mamba2_backward(ctx.shape_struct, x, dt, Ah, B, Cm, cum, D, init4, ctx.states,
                                                           dy, dfinal, ctx.has_D, ctx.has_init)
        dtd, ahd, dd, zd, wd = ctx.in_dtypes
        return (dx, ddt.to(dtd), dAh.to(ahd), dB, dC, None if dD is None else dD.to(dd), dz.reshape(ctx.z_shape).to(zd),
                dw.to(wd), None, None, None if dinit is None else dinit.reshape(ctx.init_shape))


def ssd_mamba2_gated(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor | None, z: Tensor,
                     norm_weight: Tensor, eps: float, chunk_size: int, initial_states: Tensor | None = None):
    """``rmsnorm(Y) * silu(z)`` with ``Y = SSD(x*dt, dt*A_head, B, C) + D*x``: the scan and the block's output stage
    (src/mamba_base_engine.py:170-173, :187, :189-191; norm as src/kernels/rmsnorm.py:75-150) in one operator.

    z has the size of Y ((b,T,h,p) or (b,T,h*p)); norm_weight (h*p,); the norm runs over all heads of a position.
    Returns (out in x's shape, final_state fp32 (b,h,p,n)).  Gradients: x, dt, A_head, B, C, D, z, norm_weight,
    initial_states.
    """
    return _SSDMamba2Gated.apply(x, dt, A_head, B, C, D, z, norm_weight, float(eps), int(chunk_size), initial_states)


def resolved_path_name(cfg) -> str:
    """'simt' or 'tc': the kernels the library picks for a workload configuration under the current setting."""
    lib = _cabi.load()
    shape = _cabi.Shape(_cabi.ABI_VERSION, _cabi.BF16 if cfg.dtype == "bf16" else _cabi.F32, _cabi.F32, _FORCE_PATH,
                        cfg.batch, cfg.seqlen, cfg.nheads, cfg.headdim, cfg.d_state, cfg.ngroups, cfg.chunk)
    rc = lib.ssd_b200_resolve_path(C.byref(shape))
    _cabi.check(rc)
    return {_cabi.PATH_SIMT: "simt", _cabi.PATH_TC: "tc"}[rc]
