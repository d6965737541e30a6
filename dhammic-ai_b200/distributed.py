"""Multi-GPU use of the SSD scan: one process per GPU, ``torch.distributed`` for the plumbing.

The reference has no multi-GPU path; both partitionings below build on the operator's own contract
(``initial_states`` in, ``final_state`` out, ``d final_state`` in, ``d initial_states`` out,
src/kernels/ssd_scan.py:395-397, :410, :468, :530-533).

* Batch x heads: every (batch, head) pair is an independent scan, so a rank simply runs the operator on
  its shard; nothing crosses ranks inside the operator.  Only the per-head parameter gradients
  (``dA_head``, ``dD``) are summed over ranks afterwards: :func:`allreduce_head_grads`.

* Contiguous sequence split: rank r holds positions [r*T/R, (r+1)*T/R).  The scan is linear in the
  incoming state, ``final_r = F_r + P_r * init_r`` with F_r the zero-init final state of the slice and
  P_r = exp(sum of its log-decays).  Schedule of :func:`ssd_mamba2_sequence_parallel`:

      forward   1. states-only pass over the slice            -> F_r (b,h,p,n) fp32, log P_r (b,h)
                2. all_gather of (F_r, log P_r)                 (2 MiB + 256 B per rank at h=64, p=64, n=128)
                3. init_r = sum_{q<r} (prod_{q<k<r} P_k) F_q    (local kernel over the gathered buffers)
                4. the full scan of the slice with init_r
      backward  1. dinit-only pass (reverse recurrence)         -> D_r = d init_r for a zero dfinal
                2. all_gather of (D_r, log P_r)
                3. dfinal_r = sum_{q>r} (prod_{r<k<q} P_k) D_q  (+ the caller's d final on the last rank)
                4. the full backward of the slice with init_r and dfinal_r
                5. all_reduce of dA_head and dD over the sequence group

  Gathered buffers live in this GPU's own memory and are read with plain loads.

The arithmetic is behind a small backend interface so that the communication schedule can be tested
with CPU processes over gloo (the tests plug in a CPU backend); the default backend calls the CUDA
library and fails loudly without it.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from . import _cabi
from . import ssd_scan as _op


# ----------------------------------------------------------------------------------------------------
# communicators
# ----------------------------------------------------------------------------------------------------
class TorchDistComm:
    """all_gather / all_reduce over a torch.distributed process group (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_gather(self, t: Tensor) -> Tensor:
        flat = t.contiguous().reshape(-1)
        out = torch.empty(self.world * flat.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, flat, group=self.group)
        return out.reshape((self.world,) + tuple(t.shape))

    def all_reduce_sum(self, t: Tensor) -> Tensor:
        c = t.contiguous()
        dist.all_reduce(c, op=dist.ReduceOp.SUM, group=self.group)
        return c


def allreduce_head_grads(dA_head: Tensor, dD: Tensor | None, group=None) -> None:
    """Sum the per-head parameter gradients over the ranks of a batch- or sequence-sharded group."""
    dist.all_reduce(dA_head, op=dist.ReduceOp.SUM, group=group)
    if dD is not None:
        dist.all_reduce(dD, op=dist.ReduceOp.SUM, group=group)


# ----------------------------------------------------------------------------------------------------
# the arithmetic of one rank
# ----------------------------------------------------------------------------------------------------
@dataclass
class Slice:
    """Contiguous inputs of one rank's slice of the sequence."""
    x: Tensor
    dt: Tensor
    A_head: Tensor
    B: Tensor
    C: Tensor
    D: Tensor | None
    chunk: int


class CudaBackend:
    """The per-rank passes on the CUDA library (include/ssd_b200.h)."""

    def _shape(self, s: Slice):
        return _op._make_shape(s.x, _cabi.F32, s.B, s.chunk)

    def states_only(self, s: Slice):
        """Zero-init final state of the slice and its total log-decay: (F (b,h,p,n) fp32, logp (b,h) fp32, cum)."""
        lib = _cabi.load()
        b, T, h, p = s.x.shape
        n = s.B.shape[3]
        dev = s.x.device
        shape = self._shape(s)
        with torch.cuda.device(dev):
            final = torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
            cum = torch.empty(b, h, T // s.chunk, s.chunk, dtype=torch.float32, device=dev)
            ws = _op._workspace(lib, shape, _cabi.PASS_FWD, dev)
            args = _cabi.FwdArgs(shape, _op._ptr(s.x), None, _op._ptr(s.dt), _op._ptr(s.A_head), None, _op._ptr(s.B),
                                 _op._ptr(s.C), None, None, _op._ptr(final), _op._ptr(cum), 0, _cabi.FWD_STATES_ONLY,
                                 _op._ptr(ws), ws.numel(), None)
            _cabi.check(lib.ssd_b200_fwd(C.byref(args), _op._stream(dev)))
            _op._status(lib, shape, ws, dev)
        logp = cum[..., -1].sum(-1)
        return final, logp, cum

    def forward(self, s: Slice, init: Tensor | None, cum: Tensor):
        y, final, cum, shape, states = _op._run_fwd(s.x, None, s.dt, s.A_head, s.D, s.B, s.C, s.chunk, init, None,
                                                    want_states=True)
        return y, final, {"cum": cum, "shape": shape, "states": states}

    def dinit_only(self, s: Slice, saved: dict, dy: Tensor) -> Tensor:
        lib = _cabi.load()
        b, T, h, p = s.x.shape
        dev = s.x.device
        shape = saved["shape"]
        with torch.cuda.device(dev):
            dinit = torch.empty(b, h, p, s.B.shape[3], dtype=torch.float32, device=dev)
            ws = _op._workspace(lib, shape, _cabi.PASS_BWD, dev)
            args = _cabi.BwdArgs(shape, None, None, None, None, None, None, _op._ptr(s.C), None, _op._ptr(saved["cum"]),
                                 _op._ptr(dy), None, None, None, None, None, None, None, None, _op._ptr(dinit), 0,
                                 _cabi.BWD_DINIT_ONLY, _op._ptr(ws), ws.numel(), None)
            _cabi.check(lib.ssd_b200_bwd(C.byref(args), _op._stream(dev)))
            _op._status(lib, shape, ws, dev)
        return dinit

    def backward(self, s: Slice, saved: dict, init: Tensor | None, dy: Tensor, dfinal: Tensor | None) -> dict:
        lib = _cabi.load()
        b, T, h, p = s.x.shape
        dev = s.x.device
        shape = saved["shape"]
        with torch.cuda.device(dev):
            out = {"dx": torch.empty_like(s.x), "dB": torch.empty_like(s.B), "dC": torch.empty_like(s.C),
                   "ddt": torch.empty(b, T, h, dtype=torch.float32, device=dev),
                   "dA_head": torch.empty(h, dtype=torch.float32, device=dev),
                   "dD": torch.empty(h, dtype=torch.float32, device=dev) if s.D is not None else None,
                   "dinit": torch.empty(b, h, p, s.B.shape[3], dtype=torch.float32, device=dev)}
            ws = _op._workspace(lib, shape, _cabi.PASS_BWD, dev)
            args = _cabi.BwdArgs(shape, _op._ptr(s.x), None, _op._ptr(s.dt), _op._ptr(s.A_head), _op._ptr(s.D),
                                 _op._ptr(s.B), _op._ptr(s.C), _op._ptr(init), _op._ptr(saved["cum"]), _op._ptr(dy),
                                 _op._ptr(dfinal), _op._ptr(out["dx"]), _op._ptr(out["dB"]), _op._ptr(out["dC"]), None,
                                 _op._ptr(out["ddt"]), _op._ptr(out["dA_head"]), _op._ptr(out["dD"]),
                                 _op._ptr(out["dinit"]), 0, 0, _op._ptr(ws), ws.numel(), _op._ptr(saved["states"]))
            _cabi.check(lib.ssd_b200_bwd(C.byref(args), _op._stream(dev)))
            _op._status(lib, shape, ws, dev)
        return out

    def prefix(self, states: Tensor, logp: Tensor, index: int, reverse: bool) -> Tensor:
        """states (R,b,h,p,n), logp (R,b,h) -> combination seen by position `index` (see ssd_b200_state_prefix)."""
        lib = _cabi.load()
        R, b, h, p, n = states.shape
        dev = states.device
        with torch.cuda.device(dev):
            out = torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
            _cabi.check(lib.ssd_b200_state_prefix(_op._ptr(states.contiguous()), _op._ptr(logp.contiguous()), _op._ptr(out),
                                                  R, index, b, h, p * n, 1 if reverse else 0, _op._stream(dev)))
        return out


_DEFAULT_BACKEND = CudaBackend()


class LoopbackComm:
    """A group of one: used when the sequence is only cut into segments inside a single GPU."""
    rank, world = 0, 1

    def all_gather(self, t: Tensor) -> Tensor:
        return t.unsqueeze(0)

    def all_reduce_sum(self, t: Tensor) -> Tensor:
        return t


class _SeqSplitSSD(torch.autograd.Function):
    """The scan over a sequence cut into world * S contiguous pieces: `world` ranks (one per GPU, each holding
    a contiguous slice) times S segments per rank.  The S segments of a rank run as extra batch entries of one
    launch, (b, T_rank) viewed as (b*S, T_rank/S), so that the per-(batch, head) walk kernels have enough
    blocks when b*h is small; all pieces are linked by the state prefix.  S = 1 is the plain multi-GPU
    schedule, world = 1 the split inside one GPU."""

    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, chunk, initial_state, S, comm, backend):
        b, T, h, p = x.shape
        n, g = B.shape[3], B.shape[2]
        Ts = T // S
        seg = Slice(x.contiguous().view(b * S, Ts, h, p), dt.float().contiguous().view(b * S, Ts, h),
                    A_head.float().contiguous(), B.contiguous().view(b * S, Ts, g, n),
                    C_.contiguous().view(b * S, Ts, g, n), None if D is None else D.float().contiguous(), int(chunk))
        F_loc, logp, cum = backend.states_only(seg)                              # (b*S,h,p,n), (b*S,h)
        Fs = F_loc.view(b, S, h, p, n).transpose(0, 1).contiguous()              # (S,b,h,p,n)
        lps = logp.view(b, S, h).transpose(0, 1).contiguous()                    # (S,b,h)
        allF = comm.all_gather(Fs).reshape(comm.world * S, b, h, p, n)           # piece index = rank*S + segment
        allP = comm.all_gather(lps).reshape(comm.world * S, b, h)
        init_g = torch.zeros_like(Fs[0]) if initial_state is None else initial_state.reshape(b, h, p, n).float()
        # a virtual piece in front carries the caller's initial state, so piece q sits at index q + 1
        states = torch.cat([init_g.unsqueeze(0), allF])
        lpv = torch.cat([torch.zeros_like(allP[:1]), allP])
        base = comm.rank * S
        inits = torch.stack([backend.prefix(states, lpv, base + s + 1, reverse=False) for s in range(S)], dim=1)
        inits = inits.reshape(b * S, h, p, n).contiguous()
        y, final, saved = backend.forward(seg, inits, cum)
        ctx.seg, ctx.saved, ctx.inits, ctx.allP = seg, saved, inits, allP
        ctx.comm, ctx.backend, ctx.S, ctx.dims = comm, backend, S, (b, T, h, p, n, g)
        ctx.has_init = initial_state is not None
        ctx.init_shape = None if initial_state is None else tuple(initial_state.shape)
        return y.view(b, T, h, p), final.view(b, S, h, p, n)[:, -1].contiguous()

    @staticmethod
    def backward(ctx, dy, dfinal_global):
        seg, comm, backend, S = ctx.seg, ctx.comm, ctx.backend, ctx.S
        b, T, h, p, n, g = ctx.dims
        dys = dy.contiguous().to(seg.x.dtype).view(b * S, T // S, h, p)
        Dl = backend.dinit_only(seg, ctx.saved, dys).view(b, S, h, p, n).transpose(0, 1).contiguous()
        allD = comm.all_gather(Dl).reshape(comm.world * S, b, h, p, n)
        # the caller's d final_state belongs to the last piece of the last rank: a virtual piece behind it
        extra = torch.zeros_like(Dl[0])
        if dfinal_global is not None and comm.rank == comm.world - 1:
            extra = dfinal_global.float().contiguous()
        extra = comm.all_reduce_sum(extra.clone())
        dstates = torch.cat([allD, extra.unsqueeze(0)])
        dlp = torch.cat([ctx.allP, torch.zeros_like(ctx.allP[:1])])
        base = comm.rank * S
        dfin = torch.stack([backend.prefix(dstates, dlp, base + s, reverse=True) for s in range(S)], dim=1)
        gr = backend.backward(seg, ctx.saved, ctx.inits, dys, dfin.reshape(b * S, h, p, n).contiguous())
        dAh = comm.all_reduce_sum(gr["dA_head"])
        dD = None if gr["dD"] is None else comm.all_reduce_sum(gr["dD"])
        dinit = None
        if ctx.has_init:
            d0 = gr["dinit"].view(b, S, h, p, n)[:, 0].contiguous()
            if comm.rank != 0:
                d0 = torch.zeros_like(d0)
            dinit = comm.all_reduce_sum(d0).reshape(ctx.init_shape)
        return (gr["dx"].view(b, T, h, p), gr["ddt"].view(b, T, h), dAh, gr["dB"].view(b, T, g, n),
                gr["dC"].view(b, T, g, n), dD, None, dinit, None, None, None)


def pick_segments(batch: int, nheads: int, seqlen: int, n_sm: int = 148) -> int:
    """Segments per rank so that batch*heads*segments covers the SMs about twice; 1 = no split."""
    S = 1
    while batch * nheads * S < 2 * n_sm and seqlen % (2 * S * 1024) == 0 and S < 16:
        S *= 2
    return S


def emulate_sequence_parallel(slices: list[Slice], dys: list[Tensor], initial_state: Tensor | None = None,
                              dfinal: Tensor | None = None, backend=None) -> list[dict]:
    """Run the sequence-parallel schedule for R ranks in ONE process, phase by phase over all ranks' data
    (what a box with fewer GPUs than ranks can do; also how the CUDA passes are tested on a single GPU).
    Returns one dict per rank: y, final and the gradients dx, ddt, dB, dC, dA_head, dD, dinit
    (dA_head, dD summed over ranks; dinit is the gradient of ``initial_state``)."""
    backend = backend if backend is not None else _DEFAULT_BACKEND
    R = len(slices)
    p1 = [backend.states_only(s) for s in slices]
    F = torch.stack([t[0] for t in p1])
    lp = torch.stack([t[1] for t in p1])
    init_g = torch.zeros_like(F[0]) if initial_state is None else initial_state.reshape(F[0].shape).float()
    states = torch.cat([init_g.unsqueeze(0), F])
    lps = torch.cat([torch.zeros_like(lp[:1]), lp])
    inits = [backend.prefix(states, lps, r + 1, reverse=False) for r in range(R)]
    fw = [backend.forward(s, inits[r], p1[r][2]) for r, s in enumerate(slices)]
    Dl = torch.stack([backend.dinit_only(s, fw[r][2], dys[r].contiguous()) for r, s in enumerate(slices)])
    extra = torch.zeros_like(Dl[0]) if dfinal is None else dfinal.float().contiguous()
    dstates = torch.cat([Dl, extra.unsqueeze(0)])
    dlps = torch.cat([lp, torch.zeros_like(lp[:1])])
    out = []
    for r, s in enumerate(slices):
        dfin_r = backend.prefix(dstates, dlps, r, reverse=True)
        g = backend.backward(s, fw[r][2], inits[r], dys[r].contiguous(), dfin_r)
        g["y"], g["final"] = fw[r][0], fw[r][1]
        out.append(g)
    dAh = torch.stack([g["dA_head"] for g in out]).sum(0)
    dD = None if out[0]["dD"] is None else torch.stack([g["dD"] for g in out]).sum(0)
    for g in out:
        g["dA_head"], g["dD"], g["dinit"] = dAh, dD, out[0]["dinit"]
    return out


def ssd_mamba2_sequence_parallel(x: Tensor, dt: Tensor, A_head: Tensor, B: Tensor, C: Tensor, D: Tensor | None,
                                 chunk_size: int, initial_state: Tensor | None = None, group=None, comm=None,
                                 backend=None, segments: int = 1):
    """Y = SSD(x*dt, dt*A_head, B, C) + D*x for a sequence split contiguously over the ranks of `group`.

    Every rank passes its own slice (b, T/R, ...) and the replicated per-head parameters; it gets its slice
    of Y and the final state of its slice (the last rank's is the final state of the whole sequence).
    ``initial_state`` (b,h,p,n), if given, is the state before position 0 (same tensor on every rank).
    ``dA_head`` and ``dD`` come back summed over the group.  ``segments`` > 1 additionally cuts the rank's
    slice into that many pieces run as extra batch entries (0 = choose from the shape).
    """
    comm = comm if comm is not None else TorchDistComm(group)
    backend = backend if backend is not None else _DEFAULT_BACKEND
    b, T, h, _ = x.shape
    S = segments if segments > 0 else pick_segments(b, h, T)
    if T % (S * int(chunk_size)) != 0:
        raise ValueError(f"a slice of {T} positions does not split into {S} segments of whole chunks")
    return _SeqSplitSSD.apply(x, dt, A_head, B, C, D, int(chunk_size), initial_state, S, comm, backend)


def ssd_mamba2_segmented(x, dt, A_head, B, C, D, chunk_size, initial_state=None, segments: int = 0, backend=None):
    """ssd_mamba2 with the sequence cut into `segments` pieces inside this GPU (0 = choose from the shape)."""
    return ssd_mamba2_sequence_parallel(x, dt, A_head, B, C, D, chunk_size, initial_state, comm=LoopbackComm(),
                                        backend=backend, segments=segments)
