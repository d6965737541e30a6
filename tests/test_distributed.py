"""Sequence-parallel schedule of the scan: the communication/prefix logic with two gloo processes on the
CPU (a CPU backend built on the oracle stands in for the CUDA passes), and the CUDA passes themselves on one
GPU with the ranks emulated by threads.  Both compare against the scan of the whole sequence."""
import importlib
import os
import socket
import sys
from dataclasses import replace
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from conftest import TOL_BF16, TOL_FP32, rel_err  # noqa: E402


class OracleBackend:
    """The per-rank passes on the CPU, from the oracle (test infrastructure)."""

    def __init__(self):
        from oracle import ssd_oracle
        self.O = ssd_oracle

    def _run(self, s, init):
        return self.O.mamba2_operator(s.x, s.dt, s.A_head, s.B, s.C, s.D, s.chunk,
                                      None if init is None else init.unsqueeze(1))

    def states_only(self, s, out_F=None, out_logp=None):
        with torch.no_grad():
            _, final = self._run(s, None)
        logp = (s.dt * s.A_head).sum(1)
        if out_F is not None:
            out_F.copy_(final)
            out_logp.copy_(logp)
        return final, logp, (None, None)

    def forward(self, s, init, cum):
        with torch.no_grad():
            y, final = self._run(s, init)
        return y, final, {}

    def dinit_only(self, s, saved, dy, dfinal=None, out=None):
        init0 = torch.zeros(s.x.shape[0], s.x.shape[2], s.x.shape[3], s.B.shape[3], dtype=s.x.dtype, requires_grad=True)
        with torch.enable_grad():
            y, final = self._run(s, init0)
        if dfinal is None:
            d = torch.autograd.grad([y], [init0], [dy])[0]
        else:
            d = torch.autograd.grad([y, final], [init0], [dy, dfinal])[0]
        if out is not None:
            out.copy_(d)
        return d

    def backward(self, s, saved, init, dy, dfinal):
        lv = {k: getattr(s, k).detach().clone().requires_grad_(True) for k in ("x", "dt", "A_head", "B", "C", "D")}
        il = init.detach().clone().requires_grad_(True)
        s2 = replace(s, **lv)
        with torch.enable_grad():
            y, final = self._run(s2, il)
        g = torch.autograd.grad([y, final], list(lv.values()) + [il], [dy, dfinal])
        out = {"d" + k: v for k, v in zip(lv, g[:-1])}
        out["dinit"] = g[-1]
        return out

    def prefix_all(self, pieces, logp, edge, rank, reverse, total=False, outer=None):
        R, b, S, h, p, n = pieces.shape
        P = pieces.transpose(1, 2).reshape(R * S, b, h, p, n)   # piece-major
        L = logp.transpose(1, 2).reshape(R * S, b, h)
        acc = torch.zeros_like(P[0]) if edge is None else edge.reshape(P[0].shape).to(P.dtype).clone()
        if outer is not None:   # the other ranks' whole-slice summaries first
            op, ol, orank = outer
            W = op.shape[0]
            for q in (range(W - 1, orank, -1) if reverse else range(orank)):
                acc = torch.exp(ol[q, :, 0])[..., None, None] * acc + op[q, :, 0]
        out = [None] * S
        order = range(R * S - 1, rank * S - 1, -1) if reverse else range(rank * S + S)
        lsum = torch.zeros_like(L[0])
        for g in order:
            if rank * S <= g < rank * S + S:
                out[g - rank * S] = acc
                lsum = lsum + L[g]
            acc = torch.exp(L[g])[..., None, None] * acc + P[g]
        if total:
            return acc, lsum
        return torch.stack(out, dim=1).reshape(b * S, h, p, n)


def _small_cfg(pkg):
    return replace(pkg.CONFIGS[0], batch=2, seqlen=256, nheads=4, headdim=8, d_state=16, ngroups=2, chunk=32)


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _gloo_worker(rank, world, port, result_file, segments=1):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("dhammic-ai_b200")
        D = importlib.import_module("dhammic-ai_b200.distributed")
        from oracle import ssd_oracle as O
        torch.set_num_threads(2)
        cfg = _small_cfg(pkg)
        inp = pkg.make_inputs(cfg)  # same seed on every rank: the full sequence
        g = torch.Generator().manual_seed(5)
        init = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3
        dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g)
        Tl = cfg.seqlen // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        lv = {"x": inp["x"][:, sl], "dt": inp["dt"][:, sl], "A_head": inp["A_head"], "B": inp["B"][:, sl],
              "C": inp["C"][:, sl], "D": inp["D"]}
        lv = {k: v.clone().requires_grad_(True) for k, v in lv.items()}
        il = init.clone().requires_grad_(True)
        y, final = D.ssd_mamba2_sequence_parallel(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk,
                                                  il, backend=OracleBackend(), segments=segments)
        # the caller's d final_state acts on the last rank's final state only
        outs, gouts = [y], [inp["dy"][:, sl]]
        if rank == world - 1:
            outs.append(final)
            gouts.append(dfin)
        grads = torch.autograd.grad(outs, list(lv.values()) + [il], gouts)
        got = {"y": y.detach(), "final": final.detach()}
        got.update({"d" + k: v for k, v in zip(list(lv) + ["init"], grads)})
        want = O.mamba2_fwd_bwd(inp, cfg.chunk, torch.float32, init.unsqueeze(1), dfin)
        errs = {}
        for k in ("y", "dx", "ddt", "dB", "dC"):
            errs[k] = rel_err(got[k], want[k][:, sl])
        for k in ("dA_head", "dD"):
            errs[k] = rel_err(got[k], want[k])       # summed over the group by the operator
        errs["dinit"] = rel_err(got["dinit"], want["dinit"].reshape(got["dinit"].shape))
        if rank == world - 1:
            errs["final"] = rel_err(got["final"], want["final_state"])
        bad = {k: v for k, v in errs.items() if not v < TOL_FP32}
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if not bad else f"bad {errs}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,segments", [(2, 1), (4, 1), (2, 2)])
def test_sequence_parallel_schedule_gloo(tmp_path, world, segments):
    """segments > 1: every rank also cuts its slice into segments; their summaries are folded into one state per
    rank before the exchange."""
    port = _free_port()
    res = str(tmp_path / "res")
    mp.spawn(_gloo_worker, args=(world, port, res, segments), nprocs=world, join=True)
    for r in range(world):
        assert Path(f"{res}.{r}").read_text() == "ok", Path(f"{res}.{r}").read_text()


def test_head_grad_allreduce_gloo(tmp_path):
    port = _free_port()
    res = str(tmp_path / "res")
    mp.spawn(_allreduce_worker, args=(2, port, res), nprocs=2, join=True)
    for r in range(2):
        assert Path(f"{res}.{r}").read_text() == "ok"


def _allreduce_worker(rank, world, port, result_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D = importlib.import_module("dhammic-ai_b200.distributed")
        a = torch.full((4,), float(rank + 1))
        d = torch.full((4,), 10.0 * (rank + 1))
        D.allreduce_head_grads(a, d)
        ok = torch.equal(a, torch.full((4,), 3.0)) and torch.equal(d, torch.full((4,), 30.0))
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if ok else "bad")
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("idx,world,seqlen,tol,heads_groups", [(0, 2, 512, TOL_FP32, None), (2, 2, 512, TOL_BF16, None),
                                                               (2, 4, 1024, TOL_BF16, None), (2, 2, 512, TOL_BF16, (6, 2))])
def test_sequence_parallel_cuda_passes(pkg, cabi, idx, world, seqlen, tol, heads_groups):
    """States-only / dinit-only passes, the prefix kernel and the chained full passes on the GPU (the ranks
    emulated phase by phase in this process), against one call over the whole sequence.  With 6 heads in 2 groups
    (three heads per group) the summary kernel and the reverse walk run one head per CTA instead of two."""
    D = importlib.import_module("dhammic-ai_b200.distributed")
    cfg = pkg.shrink(pkg.CONFIGS[idx], 1, seqlen)
    if heads_groups:
        cfg = replace(cfg, nheads=heads_groups[0], ngroups=heads_groups[1])
    inp = {k: v.cuda() for k, v in pkg.make_inputs(cfg).items()}
    g = torch.Generator().manual_seed(5)
    init = (torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3).cuda()
    dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g).cuda()
    names = ("x", "dt", "A_head", "B", "C", "D")
    full = {k: inp[k].clone().requires_grad_(True) for k in names}
    il = init.clone().requires_grad_(True)
    y, fs = pkg.ssd_mamba2(full["x"], full["dt"], full["A_head"], full["B"], full["C"], full["D"], cfg.chunk, il)
    gw = torch.autograd.grad([y, fs], list(full.values()) + [il], [inp["dy"], dfin])
    want = {"y": y.detach(), "final": fs.detach()}
    want.update({"d" + k: v for k, v in zip(list(names) + ["init"], gw)})

    Tl = seqlen // world
    slices, dys = [], []
    for r in range(world):
        sl = slice(r * Tl, (r + 1) * Tl)
        slices.append(D.Slice(inp["x"][:, sl].contiguous(), inp["dt"][:, sl].contiguous(), inp["A_head"],
                              inp["B"][:, sl].contiguous(), inp["C"][:, sl].contiguous(), inp["D"], cfg.chunk))
        dys.append(inp["dy"][:, sl].contiguous())
    res = D.emulate_sequence_parallel(slices, dys, init, dfin)
    torch.cuda.synchronize()
    errs = {}
    for k in ("y", "dx", "ddt", "dB", "dC"):
        errs[k] = rel_err(torch.cat([res[r][k] for r in range(world)], 1), want[k])
    for k in ("dA_head", "dD", "dinit"):
        errs[k] = rel_err(res[0][k], want[k])
    errs["final"] = rel_err(res[world - 1]["final"], want["final"])
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, errs


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_schedule_cpu(pkg, oracle, world):
    """The single-process emulation of the schedule (same phases, same prefix arithmetic) on the CPU backend."""
    D = importlib.import_module("dhammic-ai_b200.distributed")
    cfg = _small_cfg(pkg)
    inp = pkg.make_inputs(cfg)
    g = torch.Generator().manual_seed(5)
    init = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3
    dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g)
    Tl = cfg.seqlen // world
    slices = [D.Slice(inp["x"][:, r * Tl:(r + 1) * Tl], inp["dt"][:, r * Tl:(r + 1) * Tl], inp["A_head"],
                      inp["B"][:, r * Tl:(r + 1) * Tl], inp["C"][:, r * Tl:(r + 1) * Tl], inp["D"], cfg.chunk)
              for r in range(world)]
    dys = [inp["dy"][:, r * Tl:(r + 1) * Tl] for r in range(world)]
    res = D.emulate_sequence_parallel(slices, dys, init, dfin, backend=OracleBackend())
    want = oracle.mamba2_fwd_bwd(inp, cfg.chunk, torch.float32, init.unsqueeze(1), dfin)
    for k in ("y", "dx", "ddt", "dB", "dC"):
        assert rel_err(torch.cat([res[r][k] for r in range(world)], 1), want[k]) < TOL_FP32, k
    assert rel_err(res[0]["dA_head"], want["dA_head"]) < TOL_FP32
    assert rel_err(res[0]["dD"], want["dD"]) < TOL_FP32
    assert rel_err(res[0]["dinit"], want["dinit"].reshape(res[0]["dinit"].shape)) < TOL_FP32
    assert rel_err(res[world - 1]["final"], want["final_state"]) < TOL_FP32


@pytest.mark.gpu
@pytest.mark.parametrize("idx,segments,tol", [(0, 2, TOL_FP32), (2, 4, TOL_BF16)])
def test_segmented_scan_inside_one_gpu(pkg, cabi, idx, segments, tol):
    """Cutting the sequence into segments that run as extra batch entries gives the result of the plain call."""
    D = importlib.import_module("dhammic-ai_b200.distributed")
    cfg = pkg.shrink(pkg.CONFIGS[idx], 2, 1024)
    inp = {k: v.cuda() for k, v in pkg.make_inputs(cfg).items()}
    g = torch.Generator().manual_seed(6)
    init = (torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3).cuda()
    dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g).cuda()
    names = ("x", "dt", "A_head", "B", "C", "D")

    def run(fn, **kw):
        lv = {k: inp[k].clone().requires_grad_(True) for k in names}
        il = init.clone().requires_grad_(True)
        y, fs = fn(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk, il, **kw)
        gr = torch.autograd.grad([y, fs], list(lv.values()) + [il], [inp["dy"], dfin])
        out = {"y": y.detach(), "final": fs.detach()}
        out.update({"d" + k: v for k, v in zip(list(names) + ["init"], gr)})
        return out

    want = run(pkg.ssd_mamba2)
    got = run(D.ssd_mamba2_segmented, segments=segments)
    torch.cuda.synchronize()
    errs = {k: rel_err(got[k], want[k]) for k in want}
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, errs
    assert D.pick_segments(1, 64, 131072) == 8 and D.pick_segments(16, 64, 4096) == 1


# ---------------------------------------------------------------------------------------------------------
# failures made on the host: no GPU is involved, nothing hangs
# ---------------------------------------------------------------------------------------------------------
def _leaving_worker(rank, world, port, result_file):
    """Rank 1 takes part in the first step and then leaves (between steps, nothing of it in flight).  Rank 0's
    next step must end in an exception from its first collective, within the group's short timeout."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    pkg = importlib.import_module("dhammic-ai_b200")
    D = importlib.import_module("dhammic-ai_b200.distributed")
    torch.set_num_threads(2)
    cfg = _small_cfg(pkg)
    inp = pkg.make_inputs(cfg)
    Tl = cfg.seqlen // world
    sl = slice(rank * Tl, (rank + 1) * Tl)

    def step():
        return D.ssd_mamba2_sequence_parallel(inp["x"][:, sl], inp["dt"][:, sl], inp["A_head"], inp["B"][:, sl],
                                              inp["C"][:, sl], inp["D"], cfg.chunk, backend=OracleBackend())

    step()
    dist.barrier()
    outcome = "left"
    if rank == 0:
        t0 = time.time()
        try:
            step()
            outcome = "no error"
        except Exception as e:  # the collective reports the missing peer
            outcome = f"raised {type(e).__name__} after {time.time() - t0:.1f}s"
    with open(f"{result_file}.{rank}", "w") as f:
        f.write(outcome)
    if rank == 0:
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    # rank 1 simply returns: its process ends without another collective


def test_rank_that_leaves_between_steps_ends_in_an_exception(tmp_path):
    port = _free_port()
    res = str(tmp_path / "res")
    mp.spawn(_leaving_worker, args=(2, port, res), nprocs=2, join=True)
    assert Path(f"{res}.1").read_text() == "left"
    out = Path(f"{res}.0").read_text()
    assert out.startswith("raised"), out
    assert float(out.split("after ")[1].rstrip("s")) < 60.0, out


class _WrongSizeComm:
    """A communicator whose gather comes back one element short (ranks that disagree on their slice shape)."""
    rank, world = 0, 2

    def all_gather(self, flat):
        return torch.zeros(self.world * flat.numel() - 1, dtype=flat.dtype), None

    def all_reduce_sum(self, flat):
        return flat, None

    @staticmethod
    def wait(handle):
        pass


def test_wrong_sized_gathered_buffer_is_rejected(pkg):
    D = importlib.import_module("dhammic-ai_b200.distributed")
    cfg = _small_cfg(pkg)
    inp = pkg.make_inputs(cfg)
    with pytest.raises(ValueError, match="all_gather returned"):
        D.ssd_mamba2_sequence_parallel(inp["x"], inp["dt"], inp["A_head"], inp["B"], inp["C"], inp["D"], cfg.chunk,
                                       comm=_WrongSizeComm(), backend=OracleBackend())


@pytest.mark.gpu
def test_bounded_wait_that_runs_out_is_reported(pkg, cabi):
    """A wait on a barrier nothing arrives at gives up after its poll limit; the kernel returns normally, the status
    word is set and ssd_b200_device_status turns it into SSD_B200_EDEVICE.  The context stays usable afterwards."""
    import ctypes as C
    lib = cabi.load()
    ws = torch.zeros(64, dtype=torch.int32, device="cuda")
    shape = cabi.Shape(cabi.ABI_VERSION, cabi.BF16, cabi.F32, cabi.PATH_TC, 1, 256, 8, 64, 128, 1, 128)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.ssd_b200_device_status(C.byref(shape), C.c_void_p(ws.data_ptr()), stream) == 0
    cabi.check(lib.ssd_b200_selftest_bounded_wait(C.c_void_p(ws.data_ptr()), 4096, stream))
    assert lib.ssd_b200_device_status(C.byref(shape), C.c_void_p(ws.data_ptr()), stream) == cabi.EDEVICE
    assert "bounded wait" in cabi.last_error()
    with pytest.raises(RuntimeError, match="bounded wait"):
        cabi.check(cabi.EDEVICE)
    # the context is intact: a normal call still works and reports a clean status
    cfg = pkg.shrink(pkg.CONFIGS[2], 1, 256)
    inp = pkg.make_inputs(cfg)
    y, _ = pkg.ssd_mamba2(*[inp[k].cuda() for k in ("x", "dt", "A_head", "B", "C", "D")], cfg.chunk)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
