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


def _gather_with_virtual(comm, local_state: Tensor, logp: Tensor, extra: Tensor | None, extra_first: bool):
    """all_gather (state, logp) over the ranks and add one virtual rank carrying `extra` (the caller's
    initial state in front, or the caller's d final at the back) with log-decay 0."""
    states = comm.all_gather(local_state)
    lps = comm.all_gather(logp)
    if extra is None:
        extra = torch.zeros_like(local_state)
    z = torch.zeros_like(logp)
    if extra_first:
        return torch.cat([extra.unsqueeze(0), states]), torch.cat([z.unsqueeze(0), lps])
    return torch.cat([states, extra.unsqueeze(0)]), torch.cat([lps, z.unsqueeze(0)])


class _SeqParallelSSD(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, chunk, initial_state, comm, backend):
        s = Slice(x.contiguous(), dt.float().contiguous(), A_head.float().contiguous(), B.contiguous(), C_.contiguous(),
                  None if D is None else D.float().contiguous(), int(chunk))
        F_loc, logp, cum = backend.states_only(s)
        init_g = None if initial_state is None else initial_state.reshape(F_loc.shape).float()
        states, lps = _gather_with_virtual(comm, F_loc, logp, init_g, extra_first=True)
        # virtual rank 0 holds the caller's initial state, so this rank sits at index rank + 1
        init = backend.prefix(states, lps, comm.rank + 1, reverse=False)
        y, final, saved = backend.forward(s, init, cum)
        ctx.s, ctx.saved, ctx.init, ctx.logp = s, saved, init, logp
        ctx.comm, ctx.backend = comm, backend
        ctx.has_init = initial_state is not None
        ctx.init_shape = None if initial_state is None else tuple(initial_state.shape)
        return y, final

    @staticmethod
    def backward(ctx, dy, dfinal_global):
        s, comm, backend = ctx.s, ctx.comm, ctx.backend
        dy = dy.contiguous().to(s.x.dtype)
        D_loc = backend.dinit_only(s, ctx.saved, dy)
        # the caller's d final_state belongs to the last rank's final state: a virtual rank behind the last
        extra = None
        if dfinal_global is not None and comm.rank == comm.world - 1:
            extra = dfinal_global.float().contiguous()
        if extra is None:
            extra = torch.zeros_like(D_loc)
        extra = comm.all_reduce_sum(extra.clone())  # every rank needs it for its suffix combination
        states, lps = _gather_with_virtual(comm, D_loc, ctx.logp, extra, extra_first=False)
        dfinal = backend.prefix(states, lps, comm.rank, reverse=True)
        g = backend.backward(s, ctx.saved, ctx.init, dy, dfinal)
        dAh = comm.all_reduce_sum(g["dA_head"])
        dD = None if g["dD"] is None else comm.all_reduce_sum(g["dD"])
        dinit = None
        if ctx.has_init:
            # d(initial state of the whole sequence) = d init of rank 0; hand it to every rank
            d0 = g["dinit"] if comm.rank == 0 else torch.zeros_like(g["dinit"])
            dinit = comm.all_reduce_sum(d0).reshape(ctx.init_shape)
        return g["dx"], g["ddt"], dAh, g["dB"], g["dC"], dD, None, dinit, None, None


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
                                 backend=None):
    """Y = SSD(x*dt, dt*A_head, B, C) + D*x for a sequence split contiguously over the ranks of `group`.

    Every rank passes its own slice (b, T/R, ...) and the replicated per-head parameters; it gets its slice
    of Y and the final state of its slice (the last rank's is the final state of the whole sequence).
    ``initial_state`` (b,h,p,n), if given, is the state before position 0 (same tensor on every rank).
    ``dA_head`` and ``dD`` come back summed over the group.
    """
    comm = comm if comm is not None else TorchDistComm(group)
    backend = backend if backend is not None else _DEFAULT_BACKEND
    return _SeqParallelSSD.apply(x, dt, A_head, B, C, D, int(chunk_size), initial_state, comm, backend)
