"""GPU parity at the sizes that are benchmarked: the CUDA path against the CPU oracle at the full sequence
length of each configuration (batch elements are independent, so one or a few of them are enough).

  config 2   per-token shape at T = 4096 (32 tiles of decay accumulation per head), b = 1, plain and with
             an initial state and a final-state gradient
  config 1   full size, b 8 x T 2048
  config 3   T = 4096, b = 1, bf16 (rotary state angles + trapezoidal two-term form)
  config 4   the slice one GPU of eight holds (T = 16384) through the segmented scan, against the oracle
             CHAINED over segments through initial_states / final_state
             (src/kernels/ssd_scan.py:395-397, :410), and the sequence-parallel schedule with its ranks
             emulated phase by phase, also against the oracle
  fast decay the tensor-core shape with a log-decay of -4 per step: the decay across one 32-column block of the
             mask exceeds the fp32 exponent range, which the factorised mask must survive

Metric: max|a-b| / max|b| per output tensor; bar 2e-2 (bf16 inputs, fp32 accumulation); the oracle runs in fp32
on the bf16-rounded inputs.  With SSD_B200_PARITY_LOG=<file> every case appends its per-tensor errors there as a
JSON line.
"""
import importlib
import json
import os
from dataclasses import replace

import pytest
import torch

from conftest import TOL_BF16, rel_err
from test_gpu_parity import check_mamba2, mamba2_gpu

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_ANGLE_GRAD_T4096 = 4e-2


def _log(case: str, errs: dict) -> None:
    path = os.environ.get("SSD_B200_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": case, "errors": {k: float(v) for k, v in errs.items()}}) + "\n")


@pytest.mark.parametrize("states", [False, True])
def test_config2_full_sequence(pkg, cabi, oracle, states):
    cfg = pkg.shrink(pkg.CONFIGS[2], 1, 4096)
    assert pkg.resolved_path_name(cfg) == "tc"
    errs = check_mamba2(pkg, oracle, cfg, TOL_BF16, init=states, dfinal=states)
    _log(f"cfg2 b1 T4096 {'init+dfinal' if states else 'plain'}", errs)


def test_config1_full_size(pkg, cabi, oracle):
    cfg = pkg.CONFIGS[1]
    assert pkg.resolved_path_name(cfg) == "tc"
    errs = check_mamba2(pkg, oracle, cfg, TOL_BF16)
    _log("cfg1 b8 T2048 (full size)", errs)


def test_config3_full_sequence(pkg, cabi, oracle):
    cfg = pkg.shrink(pkg.CONFIGS[3], 1, 4096)
    inp = pkg.make_inputs(cfg)
    names = ("x", "dt", "A_head", "B", "C", "D", "raw_angles", "lam")
    lv = {k: inp[k].to(DEV).requires_grad_(True) for k in names}
    y = pkg.ssd_mamba3(*[lv[k] for k in names], cfg.chunk)
    grads = torch.autograd.grad([y], list(lv.values()), [inp["dy"].to(DEV)])
    torch.cuda.synchronize()
    ol = {k: inp[k].float().requires_grad_(True) for k in names}
    yo = oracle.mamba3_operator(*[ol[k] for k in names], cfg.chunk)
    go = torch.autograd.grad([yo], list(ol.values()), [inp["dy"].float()])
    errs = {"y": rel_err(y, yo)}
    for k, a, b in zip(names, grads, go):
        errs["d" + k] = rel_err(a, b)
    _log("cfg3 b1 T4096", errs)
    # d raw_angles is a suffix sum along the sequence of per-position angle gradients whose within-suffix parts cancel
    # exactly (rotating every later position by the same angle changes nothing among them); what is left of the bf16
    # rounding of the rotated operands and of their gradients does not cancel and grows with the sequence length:
    # 3e-3 at 256 positions, 2.6e-2 at 4,096.  It gets its own bar here; every other tensor meets the common one.
    bars = {k: (TOL_ANGLE_GRAD_T4096 if k == "draw_angles" else TOL_BF16) for k in errs}
    bad = {k: v for k, v in errs.items() if not v < bars[k]}
    assert not bad, errs


def _oracle_chained(oracle, inp, chunk, nseg, init, dfinal):
    """The oracle over `nseg` consecutive segments, each call starting from the final state of the one before
    (initial_states / final_state of the reference operator), under one autograd graph."""
    names = ("x", "dt", "A_head", "B", "C", "D")
    lv = {k: inp[k].detach().float().cpu().requires_grad_(True) for k in names}
    il = init.detach().float().cpu().requires_grad_(True)
    T = lv["x"].shape[1]
    L = T // nseg
    state, ys = il, []
    for s in range(nseg):
        sl = slice(s * L, (s + 1) * L)
        y, state = oracle.mamba2_operator(lv["x"][:, sl], lv["dt"][:, sl], lv["A_head"], lv["B"][:, sl], lv["C"][:, sl],
                                          lv["D"], chunk, state.unsqueeze(1))
        ys.append(y)
    y = torch.cat(ys, 1)
    g = torch.autograd.grad([y, state], list(lv.values()) + [il], [inp["dy"].float().cpu(), dfinal.float().cpu()])
    want = {"y": y.detach(), "final": state.detach()}
    want.update({"d" + k: v for k, v in zip(list(names) + ["init"], g)})
    return want


def _states(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    init = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g) * 0.3
    dfin = torch.randn(cfg.batch, cfg.nheads, cfg.headdim, cfg.d_state, generator=g)
    return init, dfin


def test_config4_slice_segmented_against_chained_oracle(pkg, cabi, oracle):
    """One GPU's slice of config 4 at eight GPUs (16,384 positions): eight segments run as batch entries of one
    launch, linked by the state prefix; the oracle is chained over four segments of 4,096 positions."""
    D = importlib.import_module("dhammic-ai_b200.distributed")
    cfg = pkg.shrink(pkg.CONFIGS[4], 1, 16384)
    inp = pkg.make_inputs(cfg)
    init, dfin = _states(cfg, 6)
    names = ("x", "dt", "A_head", "B", "C", "D")
    lv = {k: inp[k].to(DEV).requires_grad_(True) for k in names}
    il = init.to(DEV).requires_grad_(True)
    y, fs = D.ssd_mamba2_segmented(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk, il, segments=8)
    gr = torch.autograd.grad([y, fs], list(lv.values()) + [il], [inp["dy"].to(DEV), dfin.to(DEV)])
    torch.cuda.synchronize()
    got = {"y": y.detach(), "final": fs.detach()}
    got.update({"d" + k: v for k, v in zip(list(names) + ["init"], gr)})
    want = _oracle_chained(oracle, inp, cfg.chunk, 4, init, dfin)
    errs = {k: rel_err(got[k], want[k]) for k in want}
    _log("cfg4 slice b1 T16384, 8 segments in one launch vs oracle chained over 4", errs)
    bad = {k: v for k, v in errs.items() if not v < TOL_BF16}
    assert not bad, errs


def test_sequence_parallel_passes_against_oracle(pkg, cabi, oracle):
    """The sequence-parallel schedule (states-only pass, prefix, full pass and the mirrored backward) with four
    ranks emulated phase by phase on this GPU, against the oracle over the whole sequence."""
    D = importlib.import_module("dhammic-ai_b200.distributed")
    world, seqlen = 4, 4096
    cfg = pkg.shrink(pkg.CONFIGS[4], 1, seqlen)
    inp = pkg.make_inputs(cfg)
    init, dfin = _states(cfg, 5)
    dev = {k: v.to(DEV) for k, v in inp.items()}
    Tl = seqlen // world
    slices, dys = [], []
    for r in range(world):
        sl = slice(r * Tl, (r + 1) * Tl)
        slices.append(D.Slice(dev["x"][:, sl].contiguous(), dev["dt"][:, sl].contiguous(), dev["A_head"],
                              dev["B"][:, sl].contiguous(), dev["C"][:, sl].contiguous(), dev["D"], cfg.chunk))
        dys.append(dev["dy"][:, sl].contiguous())
    res = D.emulate_sequence_parallel(slices, dys, init.to(DEV), dfin.to(DEV))
    torch.cuda.synchronize()
    want = oracle.mamba2_fwd_bwd(inp, cfg.chunk, torch.float32, init.unsqueeze(1), dfin)
    errs = {}
    for k in ("y", "dx", "ddt", "dB", "dC"):
        errs[k] = rel_err(torch.cat([res[r][k] for r in range(world)], 1), want[k])
    for k in ("dA_head", "dD"):
        errs[k] = rel_err(res[0][k], want[k])
    errs["dinit"] = rel_err(res[0]["dinit"], want["dinit"].reshape(res[0]["dinit"].shape))
    errs["final"] = rel_err(res[world - 1]["final"], want["final_state"])
    _log("cfg4 shape T4096 over 4 emulated ranks vs oracle", errs)
    bad = {k: v for k, v in errs.items() if not v < TOL_BF16}
    assert not bad, errs


@pytest.mark.parametrize("per_step", [-4.0, -1.0])
def test_tensor_core_path_fast_decay(pkg, cabi, oracle, per_step):
    """bf16, p 64, n 128 (the tcgen05 kernels) with a log-decay of `per_step` at every position: at -4 the decay
    across one 32-column mask block is 128 nats, beyond what a single fp32 factor can hold; the reference clamps
    its exponents to +-20 and stays finite, and so must this path."""
    cfg = replace(pkg.shrink(pkg.CONFIGS[2], 1, 512), nheads=4, ngroups=2)
    assert pkg.resolved_path_name(cfg) == "tc"
    inp = pkg.make_inputs(cfg, seed=91)
    inp["dt"] = torch.full_like(inp["dt"], 0.1)
    inp["A_head"] = torch.full_like(inp["A_head"], per_step / 0.1)
    init, dfin = _states(cfg, 7)
    got = mamba2_gpu(pkg, inp, cfg.chunk, init, dfin)
    want = oracle.mamba2_fwd_bwd(inp, cfg.chunk, torch.float32, init.unsqueeze(1), dfin)
    for k, v in got.items():
        assert torch.isfinite(v).all(), k
    errs = {k: rel_err(got[k], want[k].reshape(got[k].shape)) for k in got}
    _log(f"tc shape, log-decay {per_step} per step", errs)
    bad = {k: v for k, v in errs.items() if not v < TOL_BF16}
    assert not bad, errs
