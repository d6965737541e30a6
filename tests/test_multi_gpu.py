"""Sequence-parallel schedule on real GPUs, one process per GPU (needs at least two; skipped otherwise): the
exchange by direct stores into the peers' memory (PeerStoreComm) and by the process group's collectives must give
the same result, and both must match one call over the whole sequence on a single GPU."""
import importlib
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from conftest import TOL_BF16, rel_err  # noqa: E402

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _worker(rank, world, port, result_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("dhammic-ai_b200")
        D = importlib.import_module("dhammic-ai_b200.distributed")
        pkg.set_check_status(True)
        cfg = pkg.shrink(pkg.CONFIGS[4], 1, 4096)
        inp = pkg.make_inputs(cfg)   # same seed on every rank: the whole sequence
        g = torch.Generator().manual_seed(5)
        init = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3
        dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g)
        Tl = cfg.seqlen // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        names = ("x", "dt", "A_head", "B", "C", "D")

        def run(comm, segments):
            lv = {k: (inp[k][:, sl] if inp[k].dim() >= 3 else inp[k]).to(dev).contiguous().requires_grad_(True) for k in names}
            il = init.to(dev).requires_grad_(True)
            y, final = D.ssd_mamba2_sequence_parallel(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk,
                                                      il, comm=comm, segments=segments)
            outs, gouts = [y], [inp["dy"][:, sl].to(dev)]
            if rank == world - 1:
                outs.append(final)
                gouts.append(dfin.to(dev))
            gr = torch.autograd.grad(outs, list(lv.values()) + [il], gouts)
            torch.cuda.synchronize(dev)
            res = {"y": y.detach(), "final": final.detach()}
            res.update({"d" + k: v for k, v in zip(list(names) + ["init"], gr)})
            return res

        peer, kind = D.make_comm()
        nccl = D.TorchDistComm()
        notes = [f"comm: {kind}"]
        bad = {}
        for segments in (1, 2):
            a = run(peer, segments)
            b = run(nccl, segments)
            for k in a:
                if not torch.equal(a[k], b[k]):
                    bad[f"S{segments} {k} peer-vs-nccl"] = rel_err(a[k], b[k])
            # against the whole sequence on this GPU alone
            full = {k: inp[k].to(dev).requires_grad_(True) for k in names}
            il = init.to(dev).requires_grad_(True)
            yf, ff = pkg.ssd_mamba2(full["x"], full["dt"], full["A_head"], full["B"], full["C"], full["D"], cfg.chunk, il)
            gf = torch.autograd.grad([yf, ff], list(full.values()) + [il], [inp["dy"].to(dev), dfin.to(dev)])
            want = {"y": yf.detach()[:, sl], "dx": gf[0][:, sl], "ddt": gf[1][:, sl], "dA_head": gf[2], "dB": gf[3][:, sl],
                    "dC": gf[4][:, sl], "dD": gf[5], "dinit": gf[6]}
            if rank == world - 1:
                want["final"] = ff.detach()
            for k, w in want.items():
                e = rel_err(a[k], w)
                if not e < TOL_BF16:
                    bad[f"S{segments} {k} vs single GPU"] = e
        if isinstance(peer, D.PeerStoreComm):
            if peer.status() != 0:
                bad["peer status"] = peer.status()
        else:
            notes.append("peer stores unavailable here: fell back to the process group")
        with open(f"{result_file}.{rank}", "w") as f:
            f.write(("ok " if not bad else f"bad {bad} ") + "; ".join(notes))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_sequence_parallel_on_two_gpus_peer_stores_and_nccl(tmp_path):
    world = 2
    port = _free_port()
    res = str(tmp_path / "res")
    mp.spawn(_worker, args=(world, port, res), nprocs=world, join=True)
    for r in range(world):
        out = Path(f"{res}.{r}").read_text()
        print(out)
        assert out.startswith("ok"), out
