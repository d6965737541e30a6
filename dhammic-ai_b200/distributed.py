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

      forward   1. summary pass over the slice (a stream)       -> F_r (b,h,p,n) fp32, log P_r (b,h)
                2. ONE all_gather of the packed (F_r | log P_r)  (2 MiB + 256 B per rank at h=64, p=64, n=128)
                3. init_r = sum_{q<r} (prod_{q<k<r} P_k) F_q    (one local kernel, every gathered piece read once)
                4. the full scan of the slice with init_r
      backward  1. reverse summary pass                          -> D_r = d init_r for a zero dfinal (the caller's
                                                                    d final_state seeds the last piece)
                2. ONE all_gather of D_r
                3. dfinal_r = sum_{q>r} (prod_{r<k<q} P_k) D_q  (one local kernel)
                4. the full backward of the slice with init_r and dfinal_r
                5. ONE all_reduce of the packed (dA_head | dD | d initial state)

  When a rank also cuts its slice into S segments (run as batch entries of one launch, see below), the segments'
  summaries are first folded into the one summary of the slice on the GPU, so that what crosses NVLink stays one
  state per rank whatever S is; the states entering the segments then come from a second local fold that starts
  from init_r.

  Each collective runs on a side stream behind the pass that produces its input, so that host work and the
  preparation kernels of the next pass (cumulative sums) are not held up by it; the kernels that need the
  gathered states wait for it through an event.  Gathered buffers live in this GPU's own memory and are read
  with plain loads.

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
    """all_gather / all_reduce of flat fp32 buffers over a torch.distributed process group (NCCL on GPUs, gloo on
    CPU).  On CUDA tensors the collective is enqueued on a side stream behind the work already queued on the
    current stream, and the current stream waits for it only when :meth:`wait` is called on the handle."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._side = None
        self.timings = None   # set to a list to record (name, start event, end event) of every collective

    def read_timings(self) -> dict[str, float]:
        """Total milliseconds per collective kind since ``timings`` was set (synchronises)."""
        out: dict[str, float] = {}
        for name, e0, e1 in self.timings or []:
            e1.synchronize()
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out

    def _side_stream(self, dev):
        if self._side is None:
            self._side = torch.cuda.Stream(dev)
        return self._side

    def _run(self, t: Tensor, fn, name: str):
        if not t.is_cuda:
            fn()
            return None
        cur = torch.cuda.current_stream(t.device)
        side = self._side_stream(t.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            rec = self.timings is not None
            if rec:
                e0 = torch.cuda.Event(enable_timing=True)
                e0.record(side)
            fn()
            ev = torch.cuda.Event(enable_timing=rec)
            ev.record(side)
            if rec:
                self.timings.append((name, e0, ev))
        return ev

    def all_gather(self, flat: Tensor):
        """flat (N,) contiguous -> (world * N,) with rank r's data at [r*N, (r+1)*N); returns (tensor, handle)."""
        if flat.dim() != 1 or not flat.is_contiguous():
            raise ValueError("all_gather takes a flat contiguous buffer")
        out = torch.empty(self.world * flat.numel(), dtype=flat.dtype, device=flat.device)
        ev = self._run(flat, lambda: dist.all_gather_into_tensor(out, flat, group=self.group), "all_gather")
        if ev is not None:
            out.record_stream(self._side)
            flat.record_stream(self._side)
        return out, ev

    def all_reduce_sum(self, flat: Tensor):
        ev = self._run(flat, lambda: dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group), "all_reduce")
        if ev is not None:
            flat.record_stream(self._side)
        return flat, ev

    @staticmethod
    def wait(handle) -> None:
        if handle is not None:
            torch.cuda.current_stream().wait_event(handle)


class PeerStoreComm(TorchDistComm):
    """all_gather of the per-rank summaries by direct stores into the other GPUs' memory over NVLink, one process per
    GPU on one node.  Every rank allocates a receive buffer (one slot per source rank, two buffers used alternately)
    and a row of arrival counters, shares them with the other processes through CUDA IPC (the handles travel
    through the process group once per buffer size; every process opens them with its own device as the accessor)
    and keeps the peers' mappings.  An
    exchange is two small launches of the library on the current stream: ``ssd_b200_exchange_push`` stores the
    block into every rank's slot, ``ssd_b200_exchange_arrive`` signals the peers and waits (bounded) for theirs.
    What was received is then read from this GPU's own memory.  No TMA, no multicast, no NCCL kernel on this path;
    the small all_reduce of the parameter gradients stays on the process group.

    ``status()`` must be checked by the caller where it matters: a wait that ran out leaves 3 there."""

    MAX_POLLS = 1 << 25

    def __init__(self, group=None):
        super().__init__(group)
        self._bufs = {}      # block size -> dict of tensors
        self._imported = {}  # IPC handle bytes -> base address of the peer allocation as mapped into this process
        self._epoch = 0
        self._dev = torch.device("cuda", torch.cuda.current_device())
        self._status = torch.zeros(1, dtype=torch.int32, device=self._dev)

    def _setup(self, n: int) -> dict:
        # one allocation per block size: [2 buffers][world slots][n floats] followed by [2][world] arrival counters
        nbuf = 2 * self.world * n
        mem = torch.zeros(nbuf + 2 * self.world, dtype=torch.float32, device=self._dev)
        torch.cuda.synchronize(self._dev)
        lib = _cabi.load()
        handle = (C.c_ubyte * 64)()
        off = C.c_int64(0)
        why = ""
        try:
            _cabi.check(lib.ssd_b200_ipc_export(_op._ptr(mem), handle, C.byref(off)))
        except Exception as e:
            why = f"{type(e).__name__}: {e}"
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (bytes(handle), int(off.value), self._dev.index, why), group=self.group)
        bases = []   # float32 base address of every rank's allocation as mapped here
        if not any(w for _, _, _, w in everyone):
            try:
                with torch.cuda.device(self._dev):   # the accessor is THIS device
                    for q, (hb, ofs, _, _) in enumerate(everyone):
                        if q == self.rank:
                            bases.append(mem.data_ptr())
                            continue
                        base = self._imported.get(hb)
                        if base is None:   # an allocation is opened once per process
                            out = C.c_void_p()
                            _cabi.check(lib.ssd_b200_ipc_import(hb, C.byref(out)))
                            base = self._imported[hb] = int(out.value)
                        bases.append(base + ofs)
            except Exception as e:   # reported to every rank below, so that all of them give up together
                why = f"{type(e).__name__}: {e}"
        else:
            why = "; ".join(w for _, _, _, w in everyone if w)
        ok = torch.tensor([0 if why else 1], device=self._dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)   # also: nobody stores before everyone has mapped
        if int(ok.item()) == 0:
            raise RuntimeError("the ranks of this group cannot map each other's device memory" + (f" ({why})" if why else ""))
        ptr_b = torch.tensor(bases, dtype=torch.int64, device=self._dev)
        ptr_f = ptr_b + 4 * nbuf
        return {"mem": mem, "buf": mem[:nbuf], "ptr_b": ptr_b,
                "ptr_f": (ptr_f, ptr_f + 4 * self.world),   # the two rows of counters (one per buffer parity) of every rank
                "epoch": 0}

    def all_gather(self, flat: Tensor):
        if not flat.is_cuda:
            return super().all_gather(flat)
        if flat.dim() != 1 or not flat.is_contiguous() or flat.dtype != torch.float32 or flat.numel() % 4:
            raise ValueError("the peer-store exchange takes a flat contiguous fp32 buffer of a multiple of 4 elements")
        n = flat.numel()
        st = self._bufs.get(n)
        if st is None:
            st = self._bufs[n] = self._setup(n)
        lib = _cabi.load()
        st["epoch"] += 1
        epoch, par = st["epoch"], st["epoch"] & 1
        stream = _op._stream(self._dev)
        rec = self.timings is not None
        if rec:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        _cabi.check(lib.ssd_b200_exchange_push(_op._ptr(flat), n, _op._ptr(st["ptr_b"]), self.world,
                                               (par * self.world + self.rank) * n, stream))
        _cabi.check(lib.ssd_b200_exchange_arrive(_op._ptr(st["ptr_f"][par]), self.rank, self.world, epoch,
                                                 _op._ptr(self._status), self.MAX_POLLS, stream))
        if rec:
            e1.record()
            self.timings.append(("peer_store_gather", e0, e1))
        return st["buf"][par * self.world * n:(par + 1) * self.world * n], None

    def status(self) -> int:
        """0, or 3 when a bounded wait for a peer ran out since the start (synchronises)."""
        return int(self._status.item())


def make_comm(group=None, prefer_peer_stores: bool = True):
    """The communicator of the sequence-parallel schedule on GPUs: direct peer stores when the ranks of the group can
    map each other's memory (one node, CUDA IPC), otherwise the process group's collectives.  Returns
    (communicator, description)."""
    if prefer_peer_stores and torch.cuda.is_available() and dist.get_backend(group) == "nccl":
        try:   # mapping is agreed on by all ranks: either every rank gets the communicator or every rank gets the exception
            comm = PeerStoreComm(group)
            comm.all_gather(torch.zeros(4, dtype=torch.float32, device=comm._dev))
            return comm, "direct stores into the peers' buffers over NVLink (CUDA IPC mappings), bounded arrival wait"
        except RuntimeError as e:
            return TorchDistComm(group), f"process-group collectives ({e})"
    return TorchDistComm(group), "process-group collectives"


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

    def states_only(self, s: Slice, out_F: Tensor | None = None, out_logp: Tensor | None = None):
        """Summary of the slice for a zero incoming state: (F (b,h,p,n) fp32, logp (b,h) fp32, cum); F and logp are
        written into ``out_F`` / ``out_logp`` when given (views of a gather buffer)."""
        lib = _cabi.load()
        b, T, h, p = s.x.shape
        n = s.B.shape[3]
        dev = s.x.device
        shape = self._shape(s)
        with torch.cuda.device(dev):
            final = out_F if out_F is not None else torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
            logp = out_logp if out_logp is not None else torch.empty(b, h, dtype=torch.float32, device=dev)
            cum = torch.empty(b, h, T // s.chunk, s.chunk, dtype=torch.float32, device=dev)
            ws = _op._workspace(lib, shape, _cabi.PASS_FWD, dev)
            # the buffer the full pass keeps its per-tile states in: this pass already fills its per-position arrays
            nbytes = int(lib.ssd_b200_states_bytes(C.byref(shape)))
            states = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
            args = _cabi.FwdArgs(shape, _op._ptr(s.x), None, _op._ptr(s.dt), _op._ptr(s.A_head), None, _op._ptr(s.B),
                                 _op._ptr(s.C), None, None, _op._ptr(final), _op._ptr(cum), 0, _cabi.FWD_STATES_ONLY,
                                 _op._ptr(ws), ws.numel(), _op._ptr(states), _op._ptr(logp))
            _cabi.check(lib.ssd_b200_fwd(C.byref(args), _op._stream(dev)))
            _op._status(lib, shape, ws, dev)
        return final, logp, (cum, states)

    def forward(self, s: Slice, init: Tensor | None, cum: Tensor):
        # the cumulative sums and per-position arrays of the summary pass are reused, not rebuilt
        cum, states = cum
        y, final, cum, shape, states = _op._run_fwd(s.x, None, s.dt, s.A_head, s.D, s.B, s.C, s.chunk, init, cum,
                                                    want_states=True, states=states, aux_valid=states is not None)
        return y, final, {"cum": cum, "shape": shape, "states": states}

    def dinit_only(self, s: Slice, saved: dict, dy: Tensor, dfinal: Tensor | None = None, out: Tensor | None = None) -> Tensor:
        """d(initial state) of the slice from dy, C and the decays alone, for the given dfinal (None = zero)."""
        lib = _cabi.load()
        b, T, h, p = s.x.shape
        dev = s.x.device
        shape = saved["shape"]
        with torch.cuda.device(dev):
            dinit = out if out is not None else torch.empty(b, h, p, s.B.shape[3], dtype=torch.float32, device=dev)
            ws = _op._workspace(lib, shape, _cabi.PASS_BWD, dev)
            args = _cabi.BwdArgs(shape, None, None, None, None, None, None, _op._ptr(s.C), None, _op._ptr(saved["cum"]),
                                 _op._ptr(dy), _op._ptr(dfinal), None, None, None, None, None, None, None,
                                 _op._ptr(dinit), 0, _cabi.BWD_DINIT_ONLY, _op._ptr(ws), ws.numel(), _op._ptr(saved.get("states")))
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

    def prefix_all(self, pieces: Tensor, logp: Tensor, edge: Tensor | None, rank: int, reverse: bool, total: bool = False,
                   outer=None):
        """pieces (R,b,S,h,p,n) and logp (R,b,S,h): summaries and total log-decays of all R*S pieces (rank-major; the
        rank dimension may be strided, the rest dense).  Returns (b*S,h,p,n): for each of rank's S pieces the state
        entering it (forward) or the state gradient leaving it (reverse); ``edge`` (b,h,p,n) is the state before the
        first piece / the gradient behind the last one.  One launch, every piece read once.  With ``total`` it returns
        instead (fold of everything walked including rank's own pieces (b,h,p,n), sum of rank's log-decays (b,h)).
        ``outer`` = (summaries (W,b,1,h,p,n), log-decays (W,b,1,h), this rank's index): whole-slice summaries of the
        other ranks, folded in before the walk (those before this rank forward, those behind it reverse)."""
        lib = _cabi.load()
        R, b, S, h, p, n = pieces.shape
        dev = pieces.device
        assert pieces[0].is_contiguous() and logp[0].is_contiguous()
        with torch.cuda.device(dev):
            ed = None if edge is None else edge.float().contiguous()
            if total:
                out = None
                tot = torch.empty(b, h, p, n, dtype=torch.float32, device=dev)
                tlp = torch.empty(b, h, dtype=torch.float32, device=dev)
            else:
                out = torch.empty(b * S, h, p, n, dtype=torch.float32, device=dev)
                tot = tlp = None
            if outer is not None:
                op, ol, orank = outer
                assert op[0].is_contiguous() and ol[0].is_contiguous()
                oargs = (_op._ptr(op), _op._ptr(ol), op.shape[0], orank, op.stride(0) if op.shape[0] > 1 else b * h * p * n,
                         ol.stride(0) if ol.shape[0] > 1 else b * h)
            else:
                oargs = (None, None, 0, 0, 0, 0)
            _cabi.check(lib.ssd_b200_state_prefix_all(
                _op._ptr(pieces), _op._ptr(logp), _op._ptr(ed), _op._ptr(out), _op._ptr(tot), _op._ptr(tlp), R, rank, S,
                b, h, p * n, pieces.stride(0) if R > 1 else b * S * h * p * n, logp.stride(0) if R > 1 else b * S * h,
                1 if reverse else 0, *oargs, _op._stream(dev)))
        return (tot, tlp) if total else out


_DEFAULT_BACKEND = CudaBackend()


class LoopbackComm:
    """A group of one: used when the sequence is only cut into segments inside a single GPU."""
    rank, world = 0, 1

    def all_gather(self, flat: Tensor):
        return flat, None

    def all_reduce_sum(self, flat: Tensor):
        return flat, None

    @staticmethod
    def wait(handle) -> None:
        pass


def _check_gathered(t: Tensor, want: int) -> None:
    """A gathered buffer of the wrong size (ranks that disagree on the shape of their slices, a communicator for a
    different group) must end in an exception here, not in a kernel reading past the buffer."""
    if t.dim() != 1 or t.numel() != want or t.dtype != torch.float32:
        raise ValueError(f"all_gather returned {tuple(t.shape)} {t.dtype}, expected ({want},) float32: the ranks of this "
                         "group do not hold slices of the same shape")


class _SeqSplitSSD(torch.autograd.Function):
    """The scan over a sequence cut into world * S contiguous pieces: `world` ranks (one per GPU, each holding
    a contiguous slice) times S segments per rank.  The S segments of a rank run as extra batch entries of one
    launch, (b, T_rank) viewed as (b*S, T_rank/S), so that the per-(batch, head) walk kernels have enough
    blocks when b*h is small; all pieces are linked by the state prefix.  S = 1 is the plain multi-GPU
    schedule, world = 1 the split inside one GPU."""

    @staticmethod
    def forward(ctx, x, dt, A_head, B, C_, D, chunk, initial_state, S, comm, backend):
        ctx.set_materialize_grads(False)
        b, T, h, p = x.shape
        n, g = B.shape[3], B.shape[2]
        Ts = T // S
        seg = Slice(x.contiguous().view(b * S, Ts, h, p), dt.float().contiguous().view(b * S, Ts, h),
                    A_head.float().contiguous(), B.contiguous().view(b * S, Ts, g, n),
                    C_.contiguous().view(b * S, Ts, g, n), None if D is None else D.float().contiguous(), int(chunk))
        # the S segment summaries (b,S,h,p,n) and their total log-decays (b,S,h) of this rank's slice
        nF, nP, nR = b * S * h * p * n, b * S * h, b * h * p * n
        pack = torch.empty(nF + nP, dtype=torch.float32, device=x.device)
        _, _, cum = backend.states_only(seg, pack[:nF].view(b * S, h, p, n), pack[nF:].view(b * S, h))
        loc_pieces, loc_logp = pack[:nF].view(1, b, S, h, p, n), pack[nF:].view(1, b, S, h)
        init_rank = None if initial_state is None else initial_state.reshape(b, h, p, n)
        rank_logp = None
        if comm.world > 1:
            # fold the segments into the one summary of the slice; only that crosses ranks
            F_rank, lp_rank = backend.prefix_all(loc_pieces, loc_logp, None, 0, reverse=False, total=True)
            gathered, hnd = comm.all_gather(torch.cat([F_rank.reshape(-1), lp_rank.reshape(-1)]))
            _check_gathered(gathered, comm.world * (nR + b * h))
            G = gathered.view(comm.world, nR + b * h)
            rank_pieces, rank_logp = G[:, :nR].view(comm.world, b, 1, h, p, n), G[:, nR:].view(comm.world, b, 1, h)
            comm.wait(hnd)
            # rank-level and segment-level prefix in one launch: the other ranks' summaries first, then the local segments
            inits = backend.prefix_all(loc_pieces, loc_logp, init_rank, 0, reverse=False,
                                       outer=(rank_pieces, rank_logp, comm.rank))
        else:
            rank_pieces = None
            inits = backend.prefix_all(loc_pieces, loc_logp, init_rank, 0, reverse=False)
        y, final, saved = backend.forward(seg, inits, cum)
        ctx.seg, ctx.saved, ctx.inits, ctx.loc_logp, ctx.rank_logp = seg, saved, inits, loc_logp, rank_logp
        ctx.comm, ctx.backend, ctx.S, ctx.dims = comm, backend, S, (b, T, h, p, n, g)
        ctx.has_init = initial_state is not None
        ctx.init_shape = None if initial_state is None else tuple(initial_state.shape)
        return y.view(b, T, h, p), final.view(b, S, h, p, n)[:, -1].contiguous()

    @staticmethod
    def backward(ctx, dy, dfinal_global):
        seg, comm, backend, S = ctx.seg, ctx.comm, ctx.backend, ctx.S
        b, T, h, p, n, g = ctx.dims
        if dy is None:
            dy = torch.zeros(b, T, h, p, dtype=seg.x.dtype, device=seg.x.device)
        dys = dy.contiguous().to(seg.x.dtype).view(b * S, T // S, h, p)
        # the caller's d final_state belongs to the last piece of the last rank: it seeds that piece's summary and is
        # that piece's own dfinal
        last = comm.rank == comm.world - 1 and dfinal_global is not None
        seed = None
        if last:
            seed = torch.zeros(b, S, h, p, n, dtype=torch.float32, device=dys.device)
            seed[:, -1] = dfinal_global.float()
            seed = seed.view(b * S, h, p, n)
        Dl = torch.empty(b * S * h * p * n, dtype=torch.float32, device=dys.device)
        backend.dinit_only(seg, ctx.saved, dys, seed, Dl.view(b * S, h, p, n))
        loc_pieces = Dl.view(1, b, S, h, p, n)
        if comm.world > 1:
            D_rank, _ = backend.prefix_all(loc_pieces, ctx.loc_logp, None, 0, reverse=True, total=True)
            gathered, hnd = comm.all_gather(D_rank.reshape(-1))
            _check_gathered(gathered, comm.world * b * h * p * n)
            comm.wait(hnd)
            dfin = backend.prefix_all(loc_pieces, ctx.loc_logp, None, 0, reverse=True,
                                      outer=(gathered.view(comm.world, b, 1, h, p, n), ctx.rank_logp, comm.rank))
        else:
            dfin = backend.prefix_all(loc_pieces, ctx.loc_logp, None, 0, reverse=True)
        if last:
            dfin.view(b, S, h, p, n)[:, -1] += dfinal_global.float()
        gr = backend.backward(seg, ctx.saved, ctx.inits, dys, dfin)
        # one all_reduce: dA_head | dD | d initial state (only rank 0's first piece carries the latter)
        parts = [gr["dA_head"].reshape(-1)]
        if gr["dD"] is not None:
            parts.append(gr["dD"].reshape(-1))
        if ctx.has_init:
            d0 = gr["dinit"].reshape(b, S, h, p, n)[:, 0].reshape(-1)
            parts.append(d0 if comm.rank == 0 else torch.zeros_like(d0))
        red, hnd = comm.all_reduce_sum(torch.cat(parts))
        comm.wait(hnd)
        dAh = red[:h]
        dD = None if gr["dD"] is None else red[h:2 * h]
        dinit = red[-b * h * p * n:].reshape(ctx.init_shape) if ctx.has_init else None
        return (gr["dx"].reshape(b, T, h, p), gr["ddt"].reshape(b, T, h), dAh, gr["dB"].reshape(b, T, g, n),
                gr["dC"].reshape(b, T, g, n), dD, None, dinit, None, None, None)


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
    b, h, p, n = p1[0][0].shape
    F = torch.stack([t[0] for t in p1]).view(R, b, 1, h, p, n)   # one segment per rank
    lp = torch.stack([t[1] for t in p1]).view(R, b, 1, h)
    edge = None if initial_state is None else initial_state.reshape(b, h, p, n)
    inits = [backend.prefix_all(F, lp, edge, r, reverse=False) for r in range(R)]
    fw = [backend.forward(s, inits[r], p1[r][2]) for r, s in enumerate(slices)]
    seeds = [None] * (R - 1) + [None if dfinal is None else dfinal.float().contiguous()]
    Dl = torch.stack([backend.dinit_only(s, fw[r][2], dys[r].contiguous(), seeds[r]) for r, s in enumerate(slices)])
    Dl = Dl.view(R, b, 1, h, p, n)
    out = []
    for r, s in enumerate(slices):
        dfin_r = backend.prefix_all(Dl, lp, None, r, reverse=True)
        if r == R - 1 and dfinal is not None:
            dfin_r = dfin_r + dfinal.float()
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
